"""Config list shared by the GPU parity tests and the CPU-side 'everything cross-compiles' test."""
from codegendemo_b200.kcg.matmul_op import default_config
from codegendemo_b200.kcg.Utils import EnumKernelDType as E

SIMT_64 = dict(KERNEL_VARIANT=1, BLOCK_SIZE_M=64, BLOCK_SIZE_N=64, BLOCK_SIZE_K=16, THREAD_SIZE_M=4, THREAD_SIZE_N=4,
               BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=2, WARP_LAYOUT_M=4, WARP_LAYOUT_N=8, WARP_SCATTER_WIDTH_A=2,
               WARP_SCATTER_WIDTH_B=4, THREAD_SCATTER_WIDTH_A=1, THREAD_SCATTER_WIDTH_B=2, GLOB_LOAD_WIDTH_A=2,
               GLOB_LOAD_WIDTH_B=2, GLOB_STORE_WIDTH=2)
SIMT_128 = dict(KERNEL_VARIANT=1, BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=16, THREAD_SIZE_M=8,
                THREAD_SIZE_N=8, BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=2, WARP_LAYOUT_M=4, WARP_LAYOUT_N=8,
                WARP_SCATTER_WIDTH_A=4, WARP_SCATTER_WIDTH_B=4, THREAD_SCATTER_WIDTH_A=4, THREAD_SCATTER_WIDTH_B=4)
# the reference's own test tile 64x48x32 / 4x6 / LSU2 (Runtime/python/kcg/test.py:20-57), on 32-wide warps
SIMT_REF_TILE = dict(KERNEL_VARIANT=1, BLOCK_SIZE_M=64, BLOCK_SIZE_N=48, BLOCK_SIZE_K=32, THREAD_SIZE_M=4,
                     THREAD_SIZE_N=6, BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=1, WARP_LAYOUT_M=4, WARP_LAYOUT_N=8,
                     WARP_SCATTER_WIDTH_A=2, WARP_SCATTER_WIDTH_B=2, THREAD_SCATTER_WIDTH_A=2,
                     THREAD_SCATTER_WIDTH_B=2, GLOB_LOAD_WIDTH_A=4, GLOB_LOAD_WIDTH_B=2, GLOB_STORE_WIDTH=2,
                     LOCAL_SPLIT_U=2, BLOCK_MAPPING=8)

# (id, M, N, K, dtype, input distribution, keys)
SEEDED = [
    ("c1_fp32_1024_tf32x3", 1024, 1024, 1024, E.float32, "uniform", dict(BLOCK_SIZE_N=128)),
    ("c1_fp32_1024_tf32x3_atrans", 1024, 1024, 1024, E.float32, "uniform", dict(BLOCK_SIZE_N=128, isATranspose=1)),
    ("c1_fp32_1024_simt", 1024, 1024, 1024, E.float32, "uniform", SIMT_128),
    ("c1_fp32_1024_simt_atrans_lsu2", 1024, 1024, 1024, E.float32, "uniform",
     dict(SIMT_64, LOCAL_SPLIT_U=2, isATranspose=1)),
    ("c1_fp32_1024_simt_noprefetch", 1024, 1024, 1024, E.float32, "uniform",
     dict(SIMT_64, SHARED_PREFETCH=0, REG_PREFETCH=0, BLOCK_MAPPING=0)),
    ("ref_shape_1024x1056x1024_simt", 1024, 1056, 1024, E.float32, "uniform", dict(SIMT_REF_TILE, isATranspose=1)),
    ("fp32_bn256_bk16", 512, 512, 512, E.float32, "uniform", dict(BLOCK_SIZE_N=256, BLOCK_SIZE_K=16, NUM_STAGES=3)),
    ("fp32_bn256_bk32_k11008", 128, 256, 11008, E.float32, "uniform", dict(BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, NUM_STAGES=2)),
    ("fp32_bk64_2stage", 256, 256, 512, E.float32, "uniform", dict(BLOCK_SIZE_N=64, BLOCK_SIZE_K=64, NUM_STAGES=2)),
    ("fp32_bm256", 512, 256, 256, E.float32, "uniform", dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=128, NUM_STAGES=2)),
    ("fp32_splitk4", 128, 256, 4096, E.float32, "uniform", dict(BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4)),
    ("bf16_1024", 1024, 1024, 1024, E.bfloat16, "normal", dict()),
    ("bf16_256x256x64_tile", 1024, 1024, 1024, E.bfloat16, "normal", dict(BLOCK_SIZE_M=256, NUM_STAGES=3)),
    ("bf16_atrans", 512, 512, 512, E.bfloat16, "normal", dict(isATranspose=1)),
    ("bf16_bk32_group0", 512, 768, 512, E.bfloat16, "normal", dict(BLOCK_SIZE_K=32, BLOCK_MAPPING=0)),
    ("bf16_bk128_bn128", 512, 512, 1024, E.bfloat16, "normal", dict(BLOCK_SIZE_K=128, BLOCK_SIZE_N=128)),
    ("bf16_bn64_uniform", 256, 320, 192, E.bfloat16, "uniform", dict(BLOCK_SIZE_N=64, NUM_STAGES=2)),
    ("bf16_splitk_skinny", 128, 4096, 4096, E.bfloat16, "normal", dict(LOCAL_SPLIT_U=4)),
    ("bf16_splitk3_uneven", 256, 512, 1280, E.bfloat16, "normal", dict(LOCAL_SPLIT_U=3)),
    ("fp16_1024", 1024, 1024, 1024, E.float16, "normal", dict()),
    ("fp16_atrans_bm256", 512, 512, 512, E.float16, "normal", dict(isATranspose=1, BLOCK_SIZE_M=256, NUM_STAGES=3)),
    # smallest problems: one tile, one K block (pipeline prologue == epilogue)
    ("bf16_one_tile_one_kblock", 128, 64, 64, E.bfloat16, "uniform", dict(BLOCK_SIZE_N=64, NUM_STAGES=2)),
    ("fp32_one_tile_one_kblock", 128, 64, 16, E.float32, "uniform", dict(BLOCK_SIZE_N=64, BLOCK_SIZE_K=16, NUM_STAGES=2)),
    ("pair_bf16_one_tile_one_kblock", 256, 128, 64, E.bfloat16, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=128, NUM_STAGES=2)),
    ("bf16_more_stages_than_kblocks", 128, 256, 128, E.bfloat16, "normal", dict(NUM_STAGES=4)),
    ("pair_bf16_tail_split", 2048, 4096, 4096, E.bfloat16, "normal", dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512)),
    # CTA-pair kernels (tcgen05 cta_group::2): BLOCK_SIZE_M is the pair's tile height
    ("pair_bf16_256", 1024, 1024, 1024, E.bfloat16, "normal", dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256)),
    ("pair_bf16_512_two_acc", 1024, 1024, 1024, E.bfloat16, "normal", dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512)),
    ("pair_bf16_512_atrans_bn128", 1024, 512, 512, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=128, isATranspose=1)),
    ("pair_fp16_256_bk32", 512, 768, 512, E.float16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_K=32, BLOCK_MAPPING=0)),
    ("pair_fp32_256", 1024, 1024, 1024, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, NUM_STAGES=3)),
    ("pair_fp32_atrans_bk16", 512, 512, 512, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=16, isATranspose=1)),
    ("pair_fp32_splitk2", 256, 512, 2048, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=16, LOCAL_SPLIT_U=2)),
    ("pair_fp32_512x128", 1024, 512, 512, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=128, BLOCK_SIZE_K=16, NUM_STAGES=4)),
    # cluster split-K (KERNEL_VARIANT 5): LOCAL_SPLIT_U CTAs of a cluster share a tile, reduce in shared memory
    ("clusterk_bf16_split4", 256, 512, 2048, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4)),
    ("clusterk_bf16_split2_bn64_bk128", 128, 256, 1024, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=64, BLOCK_SIZE_K=128, LOCAL_SPLIT_U=2)),
    ("clusterk_bf16_split4_bn256", 128, 512, 4096, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=256, LOCAL_SPLIT_U=4)),
    ("clusterk_bf16_split3_bn256", 256, 768, 1536, E.bfloat16, "normal",   # 8 column blocks dealt 3 + 3 + 2
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=256, LOCAL_SPLIT_U=3)),
    ("clusterk_bf16_split4_bn256_bk128", 128, 512, 2560, E.bfloat16, "normal",   # two stages = the exchange buffers
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128, LOCAL_SPLIT_U=4)),
    ("clusterk_fp16_split4_atrans", 256, 256, 1024, E.float16, "normal",
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4, isATranspose=1)),
    ("clusterk_bf16_uneven_k", 128, 256, 320, E.bfloat16, "uniform",   # 5 K blocks over 4 CTAs: one CTA has none
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4)),
    ("clusterk_bf16_skinny_4096", 128, 4096, 4096, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4)),
    ("clusterk_bf16_four_tile_rows_split2", 512, 2048, 2048, E.bfloat16, "normal",   # 32 tiles, 64 CTAs
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, LOCAL_SPLIT_U=2)),
    ("clusterk_fp16_split3_bn128", 128, 384, 1536, E.float16, "uniform",   # 4 column blocks dealt 2 + 1 + 1
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=3)),
    # REG_PREFETCH = 0: one accumulator buffer, no overlap of the drain with the next tile
    ("bf16_no_acc_overlap", 512, 1024, 512, E.bfloat16, "normal", dict(REG_PREFETCH=0)),
    ("pair_bf16_512_no_acc_overlap", 2048, 1024, 512, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, REG_PREFETCH=0)),
    # the two-accumulator tile that fills TMEM, several tiles per CTA pair: accumulator released in halves
    ("pair_bf16_512_half_release", 8192, 2048, 512, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, NUM_STAGES=4)),
    ("bf16_256x256_half_release_short_k", 8192, 2048, 128, E.bfloat16, "normal",
     dict(BLOCK_SIZE_M=256, NUM_STAGES=3)),
    ("pair_bf16_serpentine_raster", 2048, 2048, 512, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_MAPPING=4, RASTER_SERPENTINE=1)),
    # B stored N x K (IS_BTRANS): the NT product
    ("bf16_btrans", 256, 512, 512, E.bfloat16, "normal", dict(IS_BTRANS=1)),
    ("fp16_btrans_bk32_atrans", 256, 256, 256, E.float16, "normal", dict(IS_BTRANS=1, BLOCK_SIZE_K=32, isATranspose=1)),
    ("pair_bf16_btrans", 1024, 512, 512, E.bfloat16, "normal", dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, IS_BTRANS=1)),
    ("pair_bf16_512_btrans_splitk", 512, 512, 1024, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, IS_BTRANS=1, LOCAL_SPLIT_U=2)),
    ("naive_fp32", 256, 192, 96, E.float32, "uniform", dict(KERNEL_VARIANT=100, BLOCK_SIZE_N=64)),
    ("naive_bf16_atrans", 256, 192, 96, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=100, isATranspose=1, BLOCK_SIZE_N=64, BLOCK_SIZE_K=32)),
]

# golden fixture -> configs able to run that shape
GOLDEN = [
    ("tile_128x64x64", E.float32, dict(BLOCK_SIZE_N=64, NUM_STAGES=2)),
    ("tile_128x64x64", E.bfloat16, dict(BLOCK_SIZE_N=64, NUM_STAGES=2)),
    ("tile_128x64x64", E.float16, dict(BLOCK_SIZE_N=64, BLOCK_SIZE_K=32, NUM_STAGES=2)),
    ("tile_128x64x64", E.float32, dict(SIMT_64, LOCAL_SPLIT_U=1)),
    ("multi_256x128x96", E.float32, dict(BLOCK_SIZE_N=64, NUM_STAGES=2)),
    ("multi_256x128x96", E.float32, dict(BLOCK_SIZE_N=128, isATranspose=1, LOCAL_SPLIT_U=3)),
    ("multi_256x128x96", E.bfloat16, dict(BLOCK_SIZE_N=128, BLOCK_SIZE_K=32)),
    ("multi_256x128x96", E.float32, dict(SIMT_64, LOCAL_SPLIT_U=2, isATranspose=1)),
    ("ref_tile_64x48x32", E.float32, dict(SIMT_REF_TILE, isATranspose=1)),
    ("ref_tile_64x48x32", E.float32, dict(SIMT_REF_TILE, isATranspose=0, LOCAL_SPLIT_U=1, SHARED_PREFETCH=0)),
]
GOLDEN_SHAPES = {"tile_128x64x64": (128, 64, 64), "multi_256x128x96": (256, 128, 96), "ref_tile_64x48x32": (64, 48, 32)}

# full-size cases run the configs the bench uses (CTA-pair kernels)
BIG_FP32 = ("c2_fp32_4096", 4096, 4096, 4096, E.float32,
            dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, NUM_STAGES=3))
BIG_BF16 = ("c3_bf16_8192", 8192, 8192, 8192, E.bfloat16,
            dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, NUM_STAGES=4))
BIG_BF16_SLAB = dict(BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, NUM_STAGES=3)  # 1024-row slab: single-CTA tiles
RECT = [("c4_bf16_128x11008", 128, 11008, 11008, E.bfloat16, dict(LOCAL_SPLIT_U=4, BLOCK_SIZE_N=256)),
        ("c4_fp32_512x4096", 512, 4096, 4096, E.float32, dict(BLOCK_SIZE_N=128, LOCAL_SPLIT_U=2)),
        ("c4_bf16_2048x4096", 2048, 4096, 4096, E.bfloat16, dict())]

# The rectangular sweep in full, M in {128, 512, 2048} x N, K in {4096, 11008} (the N = K points and the two
# mixed ones: 12 shapes) x {fp32, bf16} = 24 points, and the row slabs
# of the M-sharded 32768 x 8192 x 8192 bf16 product at 1, 2, 4 and 8 GPUs: each run with the config the operator
# and the benchmark use for that shape (kernel database entry, else the rule of thumb): (id, M, N, K, dtype, dist)
TUNED_SHAPES = [(f"c4_{'fp32' if dt == E.float32 else 'bf16'}_{m}x{n}x{k}", m, n, k, dt, "uniform")
                for n in (4096, 11008) for k in (4096, 11008) for m in (128, 512, 2048)
                for dt in (E.float32, E.bfloat16)]
TUNED_SHAPES += [(f"c5_bf16_slab_{32768 // g}_rows_g{g}", 32768 // g, 8192, 8192, E.bfloat16, "normal")
                 for g in (1, 2, 4, 8)]


# fused-epilogue cases, one per kernel family and store path: (id, M, N, K, dtype, distribution, keys)
FUSED = [
    ("bf16_tma_store", 256, 512, 512, E.bfloat16, "normal", dict()),
    ("fp16_tma_store", 256, 512, 512, E.float16, "normal", dict()),
    ("bf16_pair", 1024, 512, 512, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, NUM_STAGES=4)),
    ("bf16_splitk_reduce", 256, 512, 2048, E.bfloat16, "normal", dict(LOCAL_SPLIT_U=4)),
    ("fp32_3xtf32", 256, 256, 512, E.float32, "uniform", dict(BLOCK_SIZE_N=128)),
    ("fp32_3xtf32_splitk_reduce", 128, 256, 4096, E.float32, "uniform", dict(BLOCK_SIZE_N=128, LOCAL_SPLIT_U=4)),
    ("fp32_3xtf32_pair", 512, 512, 512, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, NUM_STAGES=3)),
    ("fp32_simt", 256, 256, 256, E.float32, "uniform", SIMT_128),
    ("fp32_simt_lsu2", 256, 256, 256, E.float32, "uniform", dict(SIMT_64, LOCAL_SPLIT_U=2)),
    ("fp32_naive", 256, 192, 96, E.float32, "uniform", dict(KERNEL_VARIANT=100, BLOCK_SIZE_N=64)),
]


# batched products: (id, batch, M, N, K of one batch, dtype, distribution, keys)
BATCHED = [
    ("bf16_batch6", 6, 256, 512, 512, E.bfloat16, "normal", dict()),
    ("bf16_batch3_pair", 3, 512, 512, 1024, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, NUM_STAGES=4)),
    ("bf16_batch5_atrans", 5, 128, 256, 384, E.bfloat16, "normal", dict(isATranspose=1)),
    ("bf16_batch4_splitk", 4, 128, 256, 2048, E.bfloat16, "normal", dict(LOCAL_SPLIT_U=2)),
    ("fp16_batch2", 2, 256, 256, 256, E.float16, "normal", dict(BLOCK_SIZE_N=128)),
    ("bf16_batch3_clusterk", 3, 128, 256, 2048, E.bfloat16, "normal",   # what bmm picks for a few skinny batches
     dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, BLOCK_SIZE_K=128, LOCAL_SPLIT_U=4)),
    ("fp32_batch4_3xtf32", 4, 256, 256, 512, E.float32, "uniform", dict(BLOCK_SIZE_N=128)),
    ("fp32_batch3_3xtf32_atrans_pair", 3, 256, 512, 256, E.float32, "uniform",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, NUM_STAGES=3, isATranspose=1)),
]


# the fused all-gather with the tile the 8-GPU sharded product runs (4096-row slabs): CTA pairs, 128-wide K blocks,
# two accumulator buffers, push warps beside the epilogue; 2.25 waves of tiles here, so the stream-K tail runs too
ALLGATHER_EXTRA = [
    ("bf16_pair_256x256x128_streamk", 2304, 4096, 1024, E.bfloat16, "normal",
     dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)),
]


def all_configs():
    out = [default_config(4096, 4096, 4096, E.bfloat16, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, NUM_STAGES=3),
           default_config(256, 256, 256, E.bfloat16, KERNEL_VARIANT=101, BLOCK_SIZE_N=64),
           default_config(256, 256, 256, E.bfloat16)]
    for (_, m, n, k, dt, _, keys) in SEEDED + FUSED + ALLGATHER_EXTRA:
        out.append(default_config(m, n, k, dt, **keys))
    for (_, _, m, n, k, dt, _, keys) in BATCHED:
        out.append(default_config(m, n, k, dt, **keys))
    for (name, dt, keys) in GOLDEN:
        m, n, k = GOLDEN_SHAPES[name]
        out.append(default_config(m, n, k, dt, **keys))
    for (_, m, n, k, dt, keys) in [BIG_FP32, BIG_BF16] + RECT:
        out.append(default_config(m, n, k, dt, **keys))
    out.append(default_config(BIG_BF16[1] // 8, BIG_BF16[2], BIG_BF16[3], BIG_BF16[4], **BIG_BF16_SLAB))
    for keys in (dict(), dict(LOCAL_SPLIT_U=2), dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256)):
        out.append(default_config(512, 512, 1024, E.bfloat16, out_dtype=E.float32, **keys))  # float32 C over bf16
    from codegendemo_b200.kcg.matmul_op import tuned_config
    for (_, m, n, k, dt, _) in TUNED_SHAPES:
        out.append(tuned_config(m, n, k, dt))
    # per-rank slabs of the two-GPU fused all-gather test (tests/helpers_allgather_ranks.py)
    for keys in (dict(), dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, NUM_STAGES=4), dict(LOCAL_SPLIT_U=2),
                 dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)):
        out.append(default_config(1024, 1024, 1024, E.bfloat16, **keys))
    return out
