"""Tuning-space enumeration: ``config_gen`` and the missing ``get_cfgs``.

Mirror of Runtime/python/kcg/ConfigGenerator.py:80-126. The reference's ``config_gen`` calls
``get_cfgs``, ``read_params`` and ``getTempJsonFileName``, none of which exist in its tree; they are
written here. ``get_cfgs`` enumerates and prunes jointly, key by key, instead of filtering a full
cartesian product (3e8 raw combinations for the reference's 1024 space): a partial assignment is
dropped as soon as a rule whose keys are all bound fails.
"""
import json
import os
from typing import Callable, Dict, Iterator, List, Tuple

from codegendemo_b200.kcg.Operators.matmul import TuningSpaceChecker_Matmul
from codegendemo_b200.kcg.Utils import ConfigKeywords, PathManager, save_to_json

kw = ConfigKeywords


def read_params(path: str) -> Dict:
    with open(path, 'r') as f:
        return json.load(f)


def getTempJsonFileName(startIndex: int, endIndex: int, outDir: str) -> str:
    return f'{outDir}/tmp_json_{startIndex}_{endIndex}.json'


def _tensor_core(cfg: Dict) -> bool:
    v = cfg.get(kw.KEY_KERNEL_VARIANT, 0)
    if v in (2, 3, 4):
        return True
    if v == 1:
        return False
    return TuningSpaceChecker_Matmul.tcgen05_tile_ok(cfg)


def _per_cta(cfg: Dict) -> Dict:
    """The operand tile one CTA holds: for the CTA-pair kernels (variant 4) half the rows and half
    the B columns of the config's tile; the config itself otherwise."""
    if cfg.get(kw.KEY_KERNEL_VARIANT, 0) != 4:
        return cfg
    half = dict(cfg)
    half[kw.KEY_BLOCK_SIZE_M] = cfg[kw.KEY_BLOCK_SIZE_M] // 2
    half[kw.KEY_BLOCK_SIZE_N] = cfg[kw.KEY_BLOCK_SIZE_N] // 2
    return half


# (keys the rule reads, predicate). A rule runs once all its keys are bound.
def _rules() -> List[Tuple[Tuple[str, ...], Callable[[Dict], bool]]]:
    def divides(cfg):
        return (cfg[kw.KEY_M] % cfg[kw.KEY_BLOCK_SIZE_M] == 0 and cfg[kw.KEY_N] % cfg[kw.KEY_BLOCK_SIZE_N] == 0 and
                cfg[kw.KEY_K] % cfg[kw.KEY_BLOCK_SIZE_K] == 0)

    def warp(cfg):
        return _tensor_core(cfg) or TuningSpaceChecker_Matmul.check_warp(cfg)

    def layout_m(cfg):
        return _tensor_core(cfg) or cfg[kw.KEY_BLOCK_LAYOUT_M] * cfg[kw.KEY_WARP_LAYOUT_M] * cfg[kw.KEY_THREAD_SIZE_M] == cfg[kw.KEY_BLOCK_SIZE_M]

    def layout_n(cfg):
        return _tensor_core(cfg) or cfg[kw.KEY_BLOCK_LAYOUT_N] * cfg[kw.KEY_WARP_LAYOUT_N] * cfg[kw.KEY_THREAD_SIZE_N] == cfg[kw.KEY_BLOCK_SIZE_N]

    def scatter_a(cfg):
        if _tensor_core(cfg):
            return True
        w, t = cfg[kw.KEY_WARP_SCATTER_WIDTH_A], cfg[kw.KEY_THREAD_SCATTER_WIDTH_A]
        return t > 0 and w >= t and w % t == 0 and cfg[kw.KEY_THREAD_SIZE_M] % w == 0

    def scatter_b(cfg):
        if _tensor_core(cfg):
            return True
        w, t = cfg[kw.KEY_WARP_SCATTER_WIDTH_B], cfg[kw.KEY_THREAD_SCATTER_WIDTH_B]
        return t > 0 and w >= t and w % t == 0 and cfg[kw.KEY_THREAD_SIZE_N] % w == 0

    def shm(cfg):
        if cfg.get(kw.KEY_KERNEL_VARIANT, 0) == 4:
            return TuningSpaceChecker_Matmul.check_shm_size(_per_cta(cfg))
        return TuningSpaceChecker_Matmul.check_shm_size(cfg)

    def simt_loads(cfg):
        return _tensor_core(cfg) or TuningSpaceChecker_Matmul.check_simt_loads(cfg)

    def splitk(cfg):
        if not _tensor_core(cfg):
            return True
        return max(1, cfg[kw.KEY_LOCAL_SPLIT_U]) <= cfg[kw.KEY_K] // cfg[kw.KEY_BLOCK_SIZE_K]

    def stages(cfg):
        st = cfg.get(kw.KEY_NUM_STAGES, 0)
        if not _tensor_core(cfg) or st <= 0:
            return True
        return TuningSpaceChecker_Matmul.tcgen05_tile_ok(_per_cta(cfg), st)

    def forced_tile(cfg):
        # KERNEL_VARIANT 2/3 demands a tile the tensor-core kernel can build
        v = cfg.get(kw.KEY_KERNEL_VARIANT, 0)
        if v == 4:  # CTA pair: each CTA holds half of the tile's rows and half of its B columns
            bm, bn = cfg[kw.KEY_BLOCK_SIZE_M], cfg[kw.KEY_BLOCK_SIZE_N]
            fp32 = int(cfg.get(kw.KEY_DTYPE_A, cfg[kw.KEY_DTYPE_C])) == 4
            if bm not in (256, 512) or bn % 2 or (bm // 256) * bn > (256 if fp32 else 512):
                return False
            return TuningSpaceChecker_Matmul.tcgen05_tile_ok(_per_cta(cfg))
        return v not in (2, 3) or TuningSpaceChecker_Matmul.tcgen05_tile_ok(cfg)

    tile = (kw.KEY_BLOCK_SIZE_M, kw.KEY_BLOCK_SIZE_N, kw.KEY_BLOCK_SIZE_K, kw.KEY_DTYPE_C)
    return [
        (tile, forced_tile),
        (tile + (kw.KEY_M, kw.KEY_N, kw.KEY_K), divides),
        (tile + (kw.KEY_WARP_LAYOUT_M, kw.KEY_WARP_LAYOUT_N, kw.KEY_WARP_SIZE), warp),
        (tile + (kw.KEY_BLOCK_LAYOUT_M, kw.KEY_WARP_LAYOUT_M, kw.KEY_THREAD_SIZE_M), layout_m),
        (tile + (kw.KEY_BLOCK_LAYOUT_N, kw.KEY_WARP_LAYOUT_N, kw.KEY_THREAD_SIZE_N), layout_n),
        (tile + (kw.KEY_WARP_SCATTER_WIDTH_A, kw.KEY_THREAD_SCATTER_WIDTH_A, kw.KEY_THREAD_SIZE_M), scatter_a),
        (tile + (kw.KEY_WARP_SCATTER_WIDTH_B, kw.KEY_THREAD_SCATTER_WIDTH_B, kw.KEY_THREAD_SIZE_N), scatter_b),
        (tile + (kw.KEY_LOCAL_SPLIT_U, kw.KEY_SHARED_PREFETCH), shm),
        (tile + (kw.KEY_LOCAL_SPLIT_U, kw.KEY_K), splitk),
        (tile + (kw.KEY_THREAD_SIZE_M, kw.KEY_THREAD_SIZE_N, kw.KEY_LOCAL_SPLIT_U, kw.KEY_GLOB_LOAD_WIDTH_A,
                 kw.KEY_GLOB_LOAD_WIDTH_B, kw.KEY_GLOB_STORE_WIDTH, kw.KEY_THREAD_SCATTER_WIDTH_B,
                 kw.KEY_WARP_SCATTER_WIDTH_A, kw.KEY_WARP_SCATTER_WIDTH_B, kw.KEY_IS_A_TRANSPOSE), simt_loads),
    ], stages


def _ordered_keys(options: Dict) -> List[str]:
    """Tile and size keys first so that the cheap, high-pruning rules fire early."""
    first = [kw.KEY_DTYPE_C, kw.KEY_DTYPE_A, kw.KEY_DTYPE_B, kw.KEY_M, kw.KEY_N, kw.KEY_K, kw.KEY_KERNEL_VARIANT,
             kw.KEY_BLOCK_SIZE_M, kw.KEY_BLOCK_SIZE_N, kw.KEY_BLOCK_SIZE_K, kw.KEY_NUM_STAGES, kw.KEY_WARP_SIZE,
             kw.KEY_WARP_LAYOUT_M, kw.KEY_WARP_LAYOUT_N, kw.KEY_THREAD_SIZE_M, kw.KEY_BLOCK_LAYOUT_M,
             kw.KEY_THREAD_SIZE_N, kw.KEY_BLOCK_LAYOUT_N, kw.KEY_WARP_SCATTER_WIDTH_A, kw.KEY_THREAD_SCATTER_WIDTH_A,
             kw.KEY_WARP_SCATTER_WIDTH_B, kw.KEY_THREAD_SCATTER_WIDTH_B, kw.KEY_LOCAL_SPLIT_U,
             kw.KEY_SHARED_PREFETCH]
    keys = [k for k in first if k in options]
    keys += [k for k in options if k not in keys]
    return keys


def iter_cfgs(param_options: Dict, dedupe_tensor_core: bool = True) -> Iterator[Dict]:
    """Yields every valid config of the space described by {key: [values...]}.

    For tensor-core tiles the thread-level keys do not change the kernel; with
    ``dedupe_tensor_core`` only the first combination of them is kept per distinct kernel.
    """
    rules, stage_rule = _rules()
    keys = _ordered_keys(param_options)
    pos = {k: i for i, k in enumerate(keys)}
    # rule -> index of the last key it needs; keys absent from the space never block a rule
    fire_at: Dict[int, List[Callable]] = {}
    for needed, fn in rules:
        present = [pos[k] for k in needed if k in pos]
        if len(present) < len([k for k in needed if k in param_options]):
            continue
        if any(k not in param_options for k in needed if k not in (kw.KEY_DTYPE_A, kw.KEY_DTYPE_B)):
            continue
        fire_at.setdefault(max(present), []).append(fn)
    if kw.KEY_NUM_STAGES in pos:
        last = max(pos[k] for k in (kw.KEY_NUM_STAGES, kw.KEY_BLOCK_SIZE_M, kw.KEY_BLOCK_SIZE_N, kw.KEY_BLOCK_SIZE_K, kw.KEY_DTYPE_C))
        fire_at.setdefault(last, []).append(stage_rule)
    tc_ignored = (kw.KEY_THREAD_SIZE_M, kw.KEY_THREAD_SIZE_N, kw.KEY_WARP_SIZE, kw.KEY_BLOCK_LAYOUT_M,
                  kw.KEY_BLOCK_LAYOUT_N, kw.KEY_WARP_LAYOUT_M, kw.KEY_WARP_LAYOUT_N, kw.KEY_GLOB_LOAD_WIDTH_A,
                  kw.KEY_GLOB_LOAD_WIDTH_B, kw.KEY_WARP_SCATTER_WIDTH_A, kw.KEY_WARP_SCATTER_WIDTH_B,
                  kw.KEY_THREAD_SCATTER_WIDTH_A, kw.KEY_THREAD_SCATTER_WIDTH_B, kw.KEY_GLOB_STORE_WIDTH,
                  kw.KEY_UNROLL_NUM, kw.KEY_REG_PREFETCH, kw.KEY_LOAD_CONTINUOUS, kw.KEY_REDUCE_C_CONTINUOUS)
    seen = set()
    cfg: Dict = {}

    def rec(i: int):
        if i == len(keys):
            out = dict(cfg)
            if dedupe_tensor_core and _tensor_core(out):
                sig = tuple((k, v) for k, v in sorted(out.items()) if k not in tc_ignored)
                if sig in seen:
                    return
                seen.add(sig)
            yield out
            return
        k = keys[i]
        for v in param_options[k]:
            cfg[k] = v
            if all(fn(cfg) for fn in fire_at.get(i, ())):
                yield from rec(i + 1)
        cfg.pop(k, None)

    yield from rec(0)


def get_cfgs(tuning_cfg_file: str) -> List[Dict]:
    return list(iter_cfgs(read_params(tuning_cfg_file)))


def split_bigjson_to_temp(bigcfgs: Dict, startIndex: int, endIndex: int, outDir: str) -> str:
    outDir = outDir.rstrip('/')
    filename = getTempJsonFileName(startIndex, endIndex, outDir)
    save_to_json({'cfgs': bigcfgs['cfgs'][startIndex:endIndex]}, filename)
    return filename


def config_gen(tuning_cfg_file: str, preGeneratedJson: str, singleLength: int, cacheTuningSPaceFile: str,
               splitBigJson=True):
    """Returns ([sub-json paths], number of configs). A pre-generated combination file skips the
    enumeration; ``cacheTuningSPaceFile`` stores the enumerated space for later runs."""
    if len(preGeneratedJson) > 0:
        print(f'======== Use pre-generated json combinations {preGeneratedJson} ==========')
        combs = read_params(preGeneratedJson)
    else:
        print(f'======== Generate combinations by {tuning_cfg_file} ==========')
        combs = {'cfgs': get_cfgs(tuning_cfg_file)}
        if len(cacheTuningSPaceFile) > 0:
            with open(cacheTuningSPaceFile, 'w') as f:
                json.dump(combs, f)
    items = combs['cfgs']
    tempFileNames = []
    if splitBigJson:
        os.makedirs(PathManager.tmp_dir(), exist_ok=True)
        for i in range(0, len(items), singleLength):
            tempFileNames.append(split_bigjson_to_temp(combs, i, i + singleLength, PathManager.tmp_dir()))
    print(f"Generated {len(items)} configurations and saved subfiles Done")
    return (tempFileNames, len(items))
