"""Autotune driver: enumerate a tuning space, compile every config, time each on the GPU, keep the
top-K. Mirror of Runtime/python/kcg/testGetKernels.py (the reference's ``main``), with the same four
positional arguments and defaults that point into this package instead of a home directory.

    python -m codegendemo_b200.kcg.testGetKernels [tuning_param_file cacheTuningSpaceFile onlyGenerateCfg splitBigJson]
"""
import argparse
import os
import sys

from codegendemo_b200.kcg.ConfigGenerator import config_gen
from codegendemo_b200.kcg.KCGTask import ParallelTaskManager
from codegendemo_b200.kcg.Utils import DeviceInfo, PathManager


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("tuning_param_file", nargs="?",
                    default=os.path.join(PathManager.tuning_configs_dir(), "GEMM_configs_4096_b200.json"))
    ap.add_argument("cacheTuningSPaceFile", nargs="?", default="")
    ap.add_argument("onlyGenerateCfg", nargs="?", type=int, default=0)
    ap.add_argument("splitBigJson", nargs="?", type=int, default=1)
    ap.add_argument("--preGenerated", default="", help="use an already enumerated combination file")
    ap.add_argument("--perfPath", default="", help="prefix of the top-K result json")
    ap.add_argument("--nProcess", type=int, default=min(32, (os.cpu_count() or 8)))
    ap.add_argument("--benchmarkcnt", type=int, default=20)
    ap.add_argument("--warmupcnt", type=int, default=1)
    ap.add_argument("--keepTopNum", type=int, default=15)
    ap.add_argument("--device", type=int, default=-1)
    ap.add_argument("--startFromSubjson", default="")
    ap.add_argument("--workDir", default="")
    a = ap.parse_args(argv)
    if a.workDir:
        PathManager.set_project_dir(a.workDir)
    PathManager.init(clearPkl=True, clearTmp=True, clearCache=True)
    perfPath = a.perfPath or os.path.join(PathManager.project_dir(), "perfRecordlog")
    smallJsonLen = a.nProcess * 5
    tempfileNames, totalLen = config_gen(a.tuning_param_file, preGeneratedJson=a.preGenerated,
                                         singleLength=smallJsonLen, cacheTuningSPaceFile=a.cacheTuningSPaceFile,
                                         splitBigJson=bool(a.splitBigJson))
    print('==== config_gen Done! ==== ')
    if a.onlyGenerateCfg >= 1:
        return 0
    dev = a.device if a.device >= 0 else DeviceInfo.get_current_device()
    tm = ParallelTaskManager(totalLen, tempfileNames, perfPath, benchmarkcnt=a.benchmarkcnt, warmupcnt=a.warmupcnt,
                             devId=dev, keepTopNum=a.keepTopNum, torchDynamicLogPath='', nTorchEpsInitTest=20)
    tm.run(maxProcess=a.nProcess, startFromSubjson=a.startFromSubjson, needCompile=True, needPerfTest=True)
    print(f"top-{a.keepTopNum} results: {perfPath}_0.json")
    return 0


if __name__ == '__main__':
    sys.exit(main())
