"""Child process of test_parallel_task_manager_*: runs ParallelTaskManager with a perf stand-in that needs
no GPU. The stand-in "times" a config from its tile size and dies once to exercise the watchdog."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from codegendemo_b200.kcg.KCGTask import KernelTestResult, ParallelTaskManager, PerfTester  # noqa: E402
from codegendemo_b200.kcg.matmul_op import default_config  # noqa: E402
from codegendemo_b200.kcg.Utils import EnumKernelDType as E, PathManager  # noqa: E402


def fake_backend(kpm, inConfig, packedKernel, nBench, nWarm):
    assert os.path.exists(inConfig.hsacoPath), "compile worker must have produced the cubin"
    assert packedKernel.m_launcher.m_runtime is None, "compile workers must not load kernels"
    r = KernelTestResult(kpm)
    r.isCorrect = True
    r.torch_elapseTimeMs = 1.0
    r.kcg_elapseTimeMs = 1000.0 / (kpm.BLOCK_SIZE_N * kpm.BLOCK_SIZE_K)
    r.acc = r.torch_elapseTimeMs / r.kcg_elapseTimeMs
    return r


def perf_target(*args):
    marker = os.path.join(sys.argv[1], "crashed_once")
    if not os.path.exists(marker):
        open(marker, "w").write("x")
        os._exit(3)  # host-made failure: the perf process dies before touching any work
    PerfTester.backend = fake_backend
    PerfTester.runPerfTests(*args, pollSeconds=0.1)


if __name__ == "__main__":
    work = sys.argv[1]
    PathManager.set_project_dir(os.path.join(work, "kcg_work"))
    PathManager.init(clearPkl=True, clearTmp=True)
    cfgs = [default_config(256, 256, 256, E.bfloat16, BLOCK_SIZE_N=bn, BLOCK_SIZE_K=bk).jsonfy()
            for bn, bk in ((64, 32), (128, 64), (256, 64))]
    sub = os.path.join(PathManager.tmp_dir(), "tmp_json_0_3.json")
    json.dump({"cfgs": cfgs}, open(sub, "w"))
    tm = ParallelTaskManager(3, [sub], os.path.join(work, "perf"), benchmarkcnt=2, warmupcnt=1, devId=0, keepTopNum=2)
    tm.perfTarget = perf_target
    tm.run(maxProcess=3, needCompile=True, needPerfTest=True)
    sys.exit(0)
