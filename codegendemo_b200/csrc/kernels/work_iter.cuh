// Work decomposition shared by the tcgen05 kernels: which (output tile, K range) units a
// persistent CTA (or CTA pair) runs, in which order. Every role of a CTA walks the same
// sequence with its own iterator.
//
// Three layers, chosen by the launcher through KcgGemmParams:
//   * whole tiles           units [0, split_first_tile): one unit = one tile, all of K;
//   * even K split          every later tile is cut into split_factor equal K ranges
//                           (LOCAL_SPLIT_U > 1: all tiles);
//   * stream-K (sk_per > 0) the K blocks of the tiles from split_first_tile on are laid end
//                           to end and cut into one contiguous range of sk_per blocks per
//                           CTA, across tile borders: the last, partial wave of a persistent
//                           grid then keeps every SM busy for the same time. A tile whose
//                           blocks fall into several ranges is reduced like an even split.
// A split tile's contributors write fp32 partials to workspace slots slot0 .. slot0 + nsplit - 1
// in K order (slot0 = slot - split); the last to arrive sums them in that order.
//
// A batched product (batch_rows > 0) is the same walk over the taller matrix of all batches' rows.
//
// Tile raster (BLOCK_MAPPING, reference semantics matmul.cpp:79-86): groups of kGroup tile rows
// walk N first, so that a wave shares A and B in L2.
#pragma once
#include "gemm_params.h"

// The iterator is plain integer arithmetic; it also compiles for the host, where a CPU test walks
// every CTA's sequence and checks that the units cover each tile's K blocks exactly once.
#ifdef __CUDACC__
#define KCG_HD __host__ __device__ __forceinline__
#else
#define KCG_HD inline
#endif

// Raster variant of the translation unit (set by the compile entry; 0 unless asked for).
#ifndef KCG_SERPENTINE
#define KCG_SERPENTINE 0
#endif

namespace kcg {

struct WorkUnit {
  int m0, n0;   // origin of the output tile (m0 counts rows of the whole, possibly batched, C)
  int mcol;     // m0 within its batch: the M coordinate of an A stored K x M
  int kofs;     // batch * K: row offset of the batch's B (and of its A when stored K x M)
  int nofs;     // batch * N: row offset of the batch's B when B is stored N x K
  int tile;     // tile index in raster order
  int split;    // index of this contributor within the tile, in K order
  int nsplit;   // contributors of the tile (1 = whole K here: store C directly)
  int slot;     // workspace slot of this contributor's partial
  int kb0, kbn; // first K block and number of K blocks
};

// kSerpentine = 1: inside a group, odd tile columns walk the group's rows upwards instead of
// downwards (the reference's serpentine variant, matmul.cpp:1279-1287), so that consecutive
// tiles of the walk always share a row block of A or a column block of B.
template <int kBM, int kBN, int kGroup, int kSerpentine = 0>
struct WorkIter {
  int u, stride, first_split, factor, num_units;
  int tiles_m, tiles_n, num_kb;
  int sk_per, sk_c, sk_g0, sk_g1;
  int batch_rows, k_size, n_size;

  KCG_HD WorkIter(const KcgGemmParams& p, int unit0, int unit_stride, int tiles_m_,
                                      int tiles_n_, int num_kb_)
      : u(unit0), stride(unit_stride), first_split(p.split_first_tile),
        factor(p.split_factor > 0 ? p.split_factor : 1), tiles_m(tiles_m_), tiles_n(tiles_n_),
        num_kb(num_kb_), sk_per(p.sk_per), sk_c(unit0), batch_rows(p.batch_rows), k_size(p.K), n_size(p.N) {
    const int tiles = tiles_m * tiles_n;
    if (sk_per > 0) {
      num_units = first_split;
      const int total = (tiles - first_split) * num_kb;
      sk_g0 = sk_c * sk_per;
      sk_g1 = sk_g0 + sk_per < total ? sk_g0 + sk_per : total;
    } else {
      num_units = first_split + (tiles - first_split) * factor;
      sk_g0 = sk_g1 = 0;
    }
  }

  KCG_HD void origin(WorkUnit& w) const {
    int mb, nb;
    if constexpr (kGroup > 1) {
      const int per_group = kGroup * tiles_n;
      const int g = w.tile / per_group;
      const int first_m = g * kGroup;
      const int gsz = (tiles_m - first_m < kGroup) ? (tiles_m - first_m) : kGroup;
      const int r = w.tile - g * per_group;
      nb = r / gsz;
      const int down = r % gsz;
      mb = first_m + ((kSerpentine && (nb & 1)) ? gsz - 1 - down : down);
    } else {
      mb = w.tile / tiles_n;
      nb = w.tile - mb * tiles_n;
    }
    w.m0 = mb * kBM;
    w.n0 = nb * kBN;
    // Batched product: the batches' A and C are stacked by rows, their B (and K x M A) by K rows;
    // a batch holds a whole number of tile rows, so a tile never straddles two of them.
    const int b = batch_rows > 0 ? w.m0 / batch_rows : 0;
    w.mcol = w.m0 - b * batch_rows;
    w.kofs = b * k_size;
    w.nofs = b * n_size;
  }

  KCG_HD bool next(WorkUnit& w) {
    if (u < num_units) {
      if (u < first_split) {
        w.tile = u;
        w.split = 0;
        w.nsplit = 1;
        w.slot = 0;
      } else {
        const int v = u - first_split;
        w.tile = first_split + v / factor;
        w.split = v - (w.tile - first_split) * factor;
        w.nsplit = factor;
        w.slot = v;
      }
      const int per = (num_kb + w.nsplit - 1) / w.nsplit;
      w.kb0 = w.split * per;
      int kb1 = w.kb0 + per;
      if (kb1 > num_kb) kb1 = num_kb;
      w.kbn = (kb1 > w.kb0) ? (kb1 - w.kb0) : 0;
      origin(w);
      u += stride;
      return true;
    }
    if (sk_g0 >= sk_g1) return false;
    // stream-K: the next piece of this CTA's range, up to the end of the tile it lies in
    const int r = sk_g0 / num_kb;
    w.tile = first_split + r;
    w.kb0 = sk_g0 - r * num_kb;
    const int left_in_tile = num_kb - w.kb0, left_in_range = sk_g1 - sk_g0;
    w.kbn = left_in_tile < left_in_range ? left_in_tile : left_in_range;
    const int c_first = (r * num_kb) / sk_per;
    const int c_last = ((r + 1) * num_kb - 1) / sk_per;
    w.nsplit = c_last - c_first + 1;
    w.split = sk_c - c_first;
    w.slot = sk_c + r;  // ranges and tiles both advance along K: range index + tile index is unique and ordered
    origin(w);
    sk_g0 += w.kbn;
    return true;
  }
};

}  // namespace kcg
