// Host-side check of the kernels' work decomposition (kernels/work_iter.cuh), built and run by
// tests/test_host_logic.py. Walks every CTA's unit sequence for one plan and verifies that
//   * each tile's K blocks are covered exactly once;
//   * a tile's contributors are numbered 0..nsplit-1 in K order and all agree on nsplit;
//   * their workspace slots are slot0 + split, distinct from every other tile's, and below `slots`.
//   * a tile's contributors agree on `share` (who reduces) and share is 0 or at most nsplit;
//   * every CTA meets its split units in increasing tile order and `last` marks exactly its final unit: a CTA
//     publishes a unit's partial before it waits for that tile's other partials, so with this order a wait
//     can only depend on publications of the same or an earlier tile - no cycle.
//   * with -DKCG_SERPENTINE=1: consecutive tiles of a raster group share a row block or a column block.
// usage: work_iter_check M N K first factor sk_per grid slots units_first [batch_rows]   (tile and raster group are macros)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "work_iter.cuh"

#ifndef WIC_BM
#define WIC_BM 128
#endif
#ifndef WIC_BN
#define WIC_BN 256
#endif
#ifndef WIC_BK
#define WIC_BK 64
#endif
#ifndef WIC_GROUP
#define WIC_GROUP 8
#endif

int main(int argc, char** argv) {
  if (argc != 10 && argc != 11) return 2;  // optional last argument: rows of one batch (M is then all batches' rows)
  KcgGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = atoi(argv[1]);
  p.N = atoi(argv[2]);
  p.K = atoi(argv[3]);
  p.split_first_tile = atoi(argv[4]);
  p.split_factor = atoi(argv[5]);
  p.sk_per = atoi(argv[6]);
  const int grid = atoi(argv[7]), slots = atoi(argv[8]);
  p.split_units_first = atoi(argv[9]);
  p.batch_rows = argc == 11 ? atoi(argv[10]) : 0;
  const int tiles_m = p.M / WIC_BM, tiles_n = p.N / WIC_BN, num_kb = p.K / WIC_BK, tiles = tiles_m * tiles_n;
  std::vector<int> cover(static_cast<size_t>(tiles) * num_kb, 0);
  struct Piece { int split, nsplit, slot, kb0, kbn, share, last; };
  std::map<int, std::vector<Piece>> by_tile;
  std::map<int, int> slot_owner;
  std::map<long long, int> origin_owner;
  int shared_tiles_count = 0;
  for (int c = 0; c < grid; ++c) {
    kcg::WorkIter<WIC_BM, WIC_BN, WIC_GROUP, KCG_SERPENTINE> it(p, c, grid, tiles_m, tiles_n, num_kb);
    kcg::WorkUnit w;
    int marked_last = 1;
    size_t prev = 0;
    int prev_tile = -1, prev_split_tile = -1, prev_last = 0;
    while (it.next(w)) {
      if (prev_last) return printf("FAIL a unit follows the one marked last (CTA %d)\n", c), 1;
      prev_last = w.last;
      if (w.nsplit > 1) {
        if (w.tile <= prev_split_tile) return printf("FAIL CTA %d meets split tiles out of order\n", c), 1;
        prev_split_tile = w.tile;
      }
      if (prev_tile >= 0) by_tile[prev_tile][prev].last = 0;  // another unit follows it
      if (w.tile < 0 || w.tile >= tiles || w.kb0 < 0 || w.kb0 + w.kbn > num_kb) return printf("FAIL range\n"), 1;
      if (w.m0 % WIC_BM || w.n0 % WIC_BN || w.m0 >= p.M || w.n0 >= p.N) return printf("FAIL origin\n"), 1;
      const int b = p.batch_rows > 0 ? w.m0 / p.batch_rows : 0;
      if (w.kofs != b * p.K || w.mcol != w.m0 - b * p.batch_rows || (p.batch_rows > 0 && w.mcol + WIC_BM > p.batch_rows))
        return printf("FAIL batch offsets of tile %d\n", w.tile), 1;
      const long long key = static_cast<long long>(w.m0) * p.N + w.n0;
      if (origin_owner.count(key) && origin_owner[key] != w.tile) return printf("FAIL two tiles share an origin\n"), 1;
      origin_owner[key] = w.tile;
      for (int kb = w.kb0; kb < w.kb0 + w.kbn; ++kb) cover[static_cast<size_t>(w.tile) * num_kb + kb]++;
      by_tile[w.tile].push_back({w.split, w.nsplit, w.slot, w.kb0, w.kbn, w.share, 1});
      marked_last = w.last;
      prev_tile = w.tile;
      prev = by_tile[w.tile].size() - 1;
    }
    if (!marked_last) return printf("FAIL CTA %d: its final unit is not marked last\n", c), 1;
  }
#if KCG_SERPENTINE
  {
    // serpentine walk: consecutive tiles of the raster share a row block or a column block
    kcg::WorkIter<WIC_BM, WIC_BN, WIC_GROUP, 1> walk(p, 0, 1, tiles_m, tiles_n, num_kb);
    kcg::WorkUnit a, b;
    for (int t = 0; t + 1 < tiles; ++t) {
      a.tile = t;
      b.tile = t + 1;
      walk.origin(a);
      walk.origin(b);
      const bool same_group = (t / (WIC_GROUP * tiles_n)) == ((t + 1) / (WIC_GROUP * tiles_n));
      if (same_group && a.m0 != b.m0 && a.n0 != b.n0) return printf("FAIL serpentine jump after tile %d\n", t), 1;
    }
  }
#endif
  for (size_t i = 0; i < cover.size(); ++i)
    if (cover[i] != 1) return printf("FAIL tile %zu block %zu covered %d times\n", i / num_kb, i % num_kb, cover[i]), 1;
  if (static_cast<int>(origin_owner.size()) != tiles) return printf("FAIL raster misses tiles\n"), 1;
  for (auto& kv : by_tile) {
    auto& v = kv.second;
    const int n = v[0].nsplit;
    if (static_cast<int>(v.size()) != n) return printf("FAIL tile %d: %zu pieces, nsplit %d\n", kv.first, v.size(), n), 1;
    std::vector<int> seen(n, 0);
    int slot0 = v[0].slot - v[0].split;
    for (auto& pc : v) {
      if (pc.nsplit != n || pc.split < 0 || pc.split >= n || seen[pc.split]++) return printf("FAIL tile %d numbering\n", kv.first), 1;
      if (pc.slot - pc.split != slot0) return printf("FAIL tile %d slot0\n", kv.first), 1;
      if (pc.share != v[0].share || pc.share < 0 || pc.share > n || (n == 1 && pc.share != 0))
        return printf("FAIL tile %d share\n", kv.first), 1;
      if (pc.share > 0) shared_tiles_count++;
      if (n > 1) {
        if (pc.slot < 0 || pc.slot >= slots) return printf("FAIL slot %d outside %d\n", pc.slot, slots), 1;
        if (slot_owner.count(pc.slot)) return printf("FAIL slot %d reused\n", pc.slot), 1;
        slot_owner[pc.slot] = kv.first;
      }
    }
    // K order: split s ends where split s + 1 begins
    std::vector<Piece> ord(n);
    for (auto& pc : v) ord[pc.split] = pc;
    int at = 0;
    for (int s = 0; s < n; ++s) {
      if (ord[s].kbn > 0 && ord[s].kb0 != at) return printf("FAIL tile %d K order\n", kv.first), 1;
      at += ord[s].kbn;
    }
    if (at != num_kb) return printf("FAIL tile %d K total\n", kv.first), 1;
  }
  printf("OK tiles %d split_tiles %zu shared_pieces %d\n", tiles, slot_owner.empty() ? size_t(0) : by_tile.size(), shared_tiles_count);
  return 0;
}
