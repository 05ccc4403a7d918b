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
// With split_units_first the split units / stream-K ranges come BEFORE the whole tiles in every
// CTA's sequence: the partial tiles are then written, summed and stored by the epilogue warps while
// the main loops of the whole tiles run, and every CTA ends with an ordinary tile.
// A split tile's contributors write fp32 partials to workspace slots slot0 .. slot0 + nsplit - 1
// in K order (slot0 = slot - split); they are summed in that order. By whom: `share` = 0 - the
// last contributor to arrive sums the whole tile; `share` > 0 - contributors 0 .. share-1 wait for
// all partials and sum one share-th of the tile each. Waits cannot form a cycle: a CTA walks its
// split units in increasing tile order and publishes a unit's partial before it waits for that
// tile's other partials, so a wait only ever depends on publications of the same or an earlier
// tile. (The kernel bounds the wait all the same and hands an abandoned share to the last arriver.)
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
  int share;    // contributors 0 .. share-1 reduce a share of the tile each; 0: the last arriver reduces
  int last;     // 1: this is the last unit of the CTA (its operand ring is idle once the MMAs have retired)
  int kb0, kbn; // first K block and number of K blocks
};

// kSerpentine = 1: inside a group, odd tile columns walk the group's rows upwards instead of
// downwards (the reference's serpentine variant, matmul.cpp:1279-1287), so that consecutive
// tiles of the walk always share a row block of A or a column block of B.
template <int kBM, int kBN, int kGroup, int kSerpentine = 0>
struct WorkIter {
  static constexpr int kMaxShare = 8;  // the tile's counter word has eight bits for shares given up
  int u, stride, first_split, factor, num_units;
  int tiles_m, tiles_n, num_kb;
  int sk_per, sk_c, sk_g0, sk_g1, sk_total;
  int batch_rows, k_size, n_size;
  bool units_first;

  KCG_HD WorkIter(const KcgGemmParams& p, int unit0, int unit_stride, int tiles_m_,
                                      int tiles_n_, int num_kb_)
      : u(unit0), stride(unit_stride), first_split(p.split_first_tile),
        factor(p.split_factor > 0 ? p.split_factor : 1), tiles_m(tiles_m_), tiles_n(tiles_n_),
        num_kb(num_kb_), sk_per(p.sk_per), sk_c(unit0), batch_rows(p.batch_rows), k_size(p.K), n_size(p.N),
        units_first(p.split_units_first != 0) {
    const int tiles = tiles_m * tiles_n;
    if (sk_per > 0) {
      num_units = first_split;
      const int total = (tiles - first_split) * num_kb;
      sk_total = total;
      sk_g0 = sk_c * sk_per;
      sk_g1 = sk_g0 + sk_per < total ? sk_g0 + sk_per : total;
    } else {
      num_units = first_split + (tiles - first_split) * factor;
      sk_g0 = sk_g1 = sk_total = 0;
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

  // One piece of this CTA's stream-K range: up to the end of the tile it lies in.
  KCG_HD void sk_piece(WorkUnit& w) {
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
    // Who sums the tile: every range but the one holding the tile's last K block ends inside the
    // tile - its CTA's last unit - and takes a share; that one does too unless it carries on
    // into the next tile. When whole tiles follow the ranges (units_first) nobody waits: ranges
    // straddle tile borders, so a tile's partials arrive at different times, and the last one to
    // arrive sums the tile.
    int last_end = (c_last + 1) * sk_per;
    if (last_end > sk_total) last_end = sk_total;
    const bool hidden = units_first && first_split > 0;
    w.share = (w.nsplit > 1 && !hidden) ? w.nsplit - (last_end > (r + 1) * num_kb ? 1 : 0) : 0;
    if (w.share > kMaxShare) w.share = 0;
    w.last = (sk_g0 + w.kbn >= sk_g1 && (!units_first || u >= num_units)) ? 1 : 0;
    origin(w);
    sk_g0 += w.kbn;
  }

  KCG_HD bool next(WorkUnit& w) {
    if (units_first && sk_g0 < sk_g1) {
      sk_piece(w);
      return true;
    }
    if (u < num_units) {
      // Unit numbering: whole tiles [0, first_split), then the even split's units - or, with
      // units_first, the split units first and the whole tiles after them.
      const int nsplit_units = num_units - first_split;
      const bool whole = units_first ? u >= nsplit_units : u < first_split;
      if (whole) {
        w.tile = units_first ? u - nsplit_units : u;
        w.split = 0;
        w.nsplit = 1;
        w.slot = 0;
        w.share = 0;
      } else {
        const int v = units_first ? u : u - first_split;
        w.tile = first_split + v / factor;
        w.split = v - (w.tile - first_split) * factor;
        w.nsplit = factor;
        w.slot = v;
        // every contributor takes a share when whole tiles follow the split units (they all start
        // with the kernel), or when the unit is every contributor's last one (it is when it is the
        // first contributor's)
        const bool hidden = units_first && first_split > 0 && sk_per == 0;
        w.share = (factor > 1 && factor <= kMaxShare && (hidden || u - w.split + stride >= num_units)) ? factor : 0;
      }
      w.last = (u + stride >= num_units && (units_first || sk_g0 >= sk_g1)) ? 1 : 0;
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
    sk_piece(w);
    return true;
  }
};

}  // namespace kcg
