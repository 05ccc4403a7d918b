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
    if v in (2, 3, 4, 5):
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

    def clusterk(cfg):
        # KERNEL_VARIANT 5: a cluster of LOCAL_SPLIT_U CTAs per 128-row tile of 16-bit data; every CTA owns whole
        # 32-column blocks of the tile, and the operand ring (>= 2 stages) must hold the received slices
        if cfg.get(kw.KEY_KERNEL_VARIANT, 0) != 5:
            return True
        dt = int(cfg.get(kw.KEY_DTYPE_A, cfg[kw.KEY_DTYPE_C]))
        s, bn, bk = cfg[kw.KEY_LOCAL_SPLIT_U], cfg[kw.KEY_BLOCK_SIZE_N], cfg[kw.KEY_BLOCK_SIZE_K]
        if dt % 30 != 2 or cfg[kw.KEY_BLOCK_SIZE_M] != 128 or not 2 <= s <= 4 or bn % 64 or bn // 32 < s:
            return False
        nch = bn // 32
        recv = ((s - 1) * -(-nch // s) + nch - nch // s) * 128 * 128  # receive slots + staging of the other CTAs' blocks
        stage = (128 + bn) * bk * 2
        stages = max(2, -(-recv // stage))
        return stage * stages + 2048 <= 227 * 1024

    tile = (kw.KEY_BLOCK_SIZE_M, kw.KEY_BLOCK_SIZE_N, kw.KEY_BLOCK_SIZE_K, kw.KEY_DTYPE_C)
    return [
        (tile + (kw.KEY_LOCAL_SPLIT_U,), clusterk),
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


# ----------------------------------------------------------------------------- cost-model pre-filter
# A B200 has 148 SMs; a persistent tcgen05 launch runs one CTA (or one CTA of a pair) per SM. The model below is
# the launcher's own view of a config - how many work units it has, how many run at once, how long one takes -
# reduced to three rates: tensor throughput per SM, operand delivery per SM, operand delivery of the whole L2.
NUM_SMS = 148
SM_MFLOP_PER_US = {"16bit": 10.0, "fp32x3": 1.4, "simt": 0.4}  # useful flop per microsecond per SM
SM_LOAD_KB_PER_US = 90.0      # shared-memory fill rate one SM sustains through TMA from L2
L2_LOAD_KB_PER_US = 7500.0    # all SMs together
LAUNCH_US = 6.0               # prologue + first load + epilogue of any launch


def estimate_us(cfg: Dict) -> float:
    """Rough run time of a config from tiles, waves and bytes (no GPU needed). Only the ORDER of configs of
    one shape matters: the pre-filter keeps those within a factor of the best estimate."""
    dt = int(cfg.get(kw.KEY_DTYPE_A, cfg[kw.KEY_DTYPE_C]))
    eb = dt % 30
    M, N, K = cfg[kw.KEY_M], cfg[kw.KEY_N], cfg[kw.KEY_K]
    bm, bn, bk = cfg[kw.KEY_BLOCK_SIZE_M], cfg[kw.KEY_BLOCK_SIZE_N], cfg[kw.KEY_BLOCK_SIZE_K]
    variant = cfg.get(kw.KEY_KERNEL_VARIANT, 0)
    split = max(1, cfg.get(kw.KEY_LOCAL_SPLIT_U, 1))
    tiles = (M // bm) * (N // bn)
    tc = _tensor_core(cfg) or variant == 5
    if not tc:
        # SIMT: one CTA per tile, LOCAL_SPLIT_U splits K inside the CTA; several CTAs share an SM
        per_sm = max(1, min(8, (200 * 1024) // max(1, (bm + bn) * bk * eb * 2)))
        waves = -(-tiles // (NUM_SMS * per_sm))
        return LAUNCH_US + waves * per_sm * 2.0 * bm * bn * K / 1e6 / SM_MFLOP_PER_US["simt"]
    pair = variant == 4
    rows, cols = (bm // 2, bn // 2) if pair else (bm, bn)   # operand slices one CTA loads
    rate = SM_MFLOP_PER_US["fp32x3" if eb == 4 else "16bit"]
    units = tiles * split                                     # a unit keeps one CTA (pair) busy
    at_once = (NUM_SMS // 2) if pair else NUM_SMS
    if variant == 5:
        units, at_once = tiles, NUM_SMS // split              # clusters of `split` CTAs, one tile each
    kb = K / bk / split
    unit_kb = (rows + cols) * bk * eb * kb / 1024.0
    unit_us = max(2.0 * rows * bn * (K / split) / 1e6 / rate, unit_kb / SM_LOAD_KB_PER_US)
    waves = units / at_once
    if waves > 1.0 and split == 1:
        waves = max(1.0, waves)                               # at best the remainder split levels the last wave
    else:
        waves = float(-(-units // at_once))
    ctas = units * (2 if pair else 1) * (split if variant == 5 else 1)
    l2_us = ctas * unit_kb / L2_LOAD_KB_PER_US
    reduce_us = 0.0
    if split > 1:
        reduce_us = 2.0 if variant == 5 else 5.0 + 0.18 * rows * bn * 4 / 1024.0
    return LAUNCH_US + max(waves * unit_us, l2_us) + reduce_us


def prefilter_by_cost(cfgs: List[Dict], keep_within: float) -> List[Dict]:
    """Keeps the configs whose estimate is within `keep_within` times the best estimate of their shape and
    type: tiles that leave most SMs idle, or re-read the operands many times over, are not worth a compile."""
    best: Dict[Tuple, float] = {}
    est = []
    for c in cfgs:
        key = (c[kw.KEY_M], c[kw.KEY_N], c[kw.KEY_K], int(c.get(kw.KEY_DTYPE_A, c[kw.KEY_DTYPE_C])))
        e = estimate_us(c)
        est.append((key, e))
        best[key] = min(best.get(key, e), e)
    return [c for c, (key, e) in zip(cfgs, est) if e <= keep_within * best[key]]


def get_cfgs(tuning_cfg_file: str) -> List[Dict]:
    """The valid configs of a tuning-space JSON. An optional entry "COST_PREFILTER": [f] (not a tuning key) keeps
    only the configs whose estimated run time is within f times the best estimate (see estimate_us)."""
    space = read_params(tuning_cfg_file)
    keep = space.pop("COST_PREFILTER", None)
    cfgs = list(iter_cfgs(space))
    if keep:
        cfgs = prefilter_by_cost(cfgs, float(keep[0] if isinstance(keep, (list, tuple)) else keep))
    return cfgs


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
