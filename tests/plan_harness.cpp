// CPU simulation of the flash-decode work partition (csrc/flash_decode_plan.h), compiled by
// tests/test_decode_plan.py with g++ and driven through ctypes.  It replays, for every CTA and warp,
// the walk the kernel makes over its column range and checks the invariants the kernel relies on:
//   * every tile of every (sequence, kv head) unit is visited exactly once;
//   * a unit is finished either by one direct write, or by exactly (last_cta - first_cta + 1) records
//     whose indices are the ones the merging warp will enumerate, and no record index is used twice;
//   * the tile loads a warp issues ahead (kStages deep) are the tiles it later consumes, in order.
#include <cstdint>
#include <map>
#include <set>
#include <vector>

#include "flash_decode_plan.h"

using namespace l3ci;

extern "C" {

int plan_tile_tokens(int D) { return fd_tile_tokens(D); }
int plan_head_group(int Hkv) { return fd_head_group(Hkv); }
int plan_max_ctas(int sms, int hg) { return fd_max_ctas(sms, hg); }
int plan_range_begin(int cta, int total, int ctas) { return fd_range_begin(cta, total, ctas); }
int plan_cta_of(int col, int total, int ctas) { return fd_cta_of(col, total, ctas); }

// Static deal: out = {W, C, ctas}; returns whether the call goes to the static kernel.
int plan_static(int B, int Hq, int Hkv, int D, int n_seq, int ragged, int sms, const int* max_clusters, int* out) {
  const long long units = (long long)B * Hkv;
  const long long tiles = ((long long)n_seq + fd_tile_tokens(D) - 1) / fd_tile_tokens(D);
  const FdStaticSplit s = fd_static_split(units, tiles, sms, max_clusters);
  out[0] = s.W; out[1] = s.C; out[2] = s.ctas;
  return fd_static_applies(s, units, tiles, D, n_seq, Hq / Hkv, ragged != 0) ? 1 : 0;
}

// Returns 0 if all invariants hold, else a positive code; info[0..3] receive details.
// stats[0] = units finished directly, stats[1] = units merged, stats[2] = records written,
// stats[3] = max columns of a CTA, stats[4] = min columns of a non-empty CTA, stats[5] = total columns,
// stats[6] = 1 if the whole-unit cut was chosen.
int plan_simulate(int B, int Hkv, int D, int n_seq, const int* seq_lens, int G, int stages, int* info,
                  long long* stats) {
  const int tile = fd_tile_tokens(D);
  const int HG = fd_head_group(Hkv);
  const int n_groups = Hkv / HG;
  std::vector<int> lens, pref;
  FdWalker wk;
  wk.B = B; wk.n_groups = n_groups; wk.n_seq = n_seq; wk.tile = tile; wk.pref = nullptr; wk.lens = nullptr;
  if (seq_lens) {
    lens.resize(B);
    pref.assign(B + 1, 0);
    for (int b = 0; b < B; ++b) {
      int l = seq_lens[b];
      l = l < 0 ? 0 : (l > n_seq ? n_seq : l);
      lens[b] = l;
      pref[b + 1] = pref[b] + n_groups * fd_tiles(l, tile);
    }
    wk.pref = pref.data();
    wk.lens = lens.data();
  }
  const int total = wk.total();
  const int grid = G;
  const int units = B * n_groups;
  const bool whole = fd_whole_units(total, units, grid);
  G = whole ? (grid < units ? grid : units) : fd_active_ctas(grid, total);
  auto unit_col = [&](int u) {
    const int b = u / n_groups, g = u - b * n_groups;
    return b >= B ? total : wk.pref_of(b) + g * fd_tiles(wk.len_of(b), tile);
  };
  stats[6] = whole;
  stats[5] = total;
  stats[3] = 0;
  stats[4] = total + 1;

  std::map<std::pair<int, int>, std::vector<int>> visited;   // (b, head) -> tile visit counts
  std::map<std::pair<int, int>, int> direct, arrivals, expected;
  std::map<std::pair<int, int>, std::set<int>> unit_records;
  std::set<int> all_records;
  long long n_records = 0;

  for (int cta = 0; cta < G; ++cta) {
    const int c0 = whole ? unit_col(fd_range_begin(cta, units, G)) : fd_range_begin(cta, total, G);
    const int c1 = whole ? unit_col(fd_range_begin(cta + 1, units, G)) : fd_range_begin(cta + 1, total, G);
    if (c0 >= c1) { info[0] = cta; return 1; }  // every active CTA owns a column
    if (c1 - c0 > stats[3]) stats[3] = c1 - c0;
    if (c1 - c0 < stats[4]) stats[4] = c1 - c0;
    for (int col = c0; col < c1 && !whole; ++col)
      if (fd_cta_of(col, total, G) != cta) { info[0] = cta; info[1] = col; info[2] = fd_cta_of(col, total, G); return 2; }
    for (int warp = 0; warp < HG; ++warp) {
      FdCursor prod = wk.seek(c0), cons = prod;
      std::vector<FdCursor> inflight;
      for (int s = 0; s < stages; ++s)
        if (prod.col < c1) { inflight.push_back(prod); wk.advance(prod); }
      size_t next = 0;
      while (cons.col < c1) {
        const int head = cons.g * HG + warp;
        // the tile being consumed must be the oldest issued one
        if (next >= inflight.size()) { info[0] = cta; info[1] = cons.col; return 3; }
        const FdCursor& is = inflight[next++];
        if (is.b != cons.b || is.g != cons.g || is.j != cons.j) { info[0] = cta; info[1] = cons.col; return 4; }
        if (cons.b < 0 || cons.b >= B || head >= Hkv || cons.j < 0 || cons.j >= cons.tc) { info[0] = cta; info[1] = cons.col; return 5; }
        if (cons.len != (seq_lens ? lens[cons.b] : n_seq) || cons.tc != fd_tiles(cons.len, tile)) { info[0] = cta; return 6; }
        auto& vis = visited[{cons.b, head}];
        if (vis.empty()) vis.assign(cons.tc, 0);
        vis[cons.j]++;
        if (prod.col < c1) { inflight.push_back(prod); wk.advance(prod); }
        if (fd_unit_ends(cons, c1)) {
          const int u0 = wk.unit_begin(cons);
          const int cfirst = whole ? cta : fd_cta_of(u0, total, G), clast = whole ? cta : fd_cta_of(u0 + cons.tc - 1, total, G);
          if (whole && (u0 < c0 || u0 + cons.tc > c1)) { info[0] = cta; info[1] = u0; return 16; }  // unit not whole
          if (cta < cfirst || cta > clast) { info[0] = cta; info[1] = cfirst; info[2] = clast; return 7; }
          if (cfirst == clast) {
            direct[{cons.b, head}]++;
          } else {
            const int rec = fd_record_index(cta, cfirst, HG, warp);
            if (rec < 0 || rec >= grid * 2 * HG) { info[0] = cta; info[1] = rec; return 8; }
            if (!all_records.insert(rec).second) { info[0] = cta; info[1] = rec; return 9; }
            unit_records[{cons.b, head}].insert(rec);
            arrivals[{cons.b, head}]++;
            expected[{cons.b, head}] = clast - cfirst + 1;
            ++n_records;
            // what the merging warp would read
            std::set<int> want;
            for (int c = cfirst; c <= clast; ++c) want.insert(fd_record_index(c, cfirst, HG, warp));
            if (arrivals[{cons.b, head}] == clast - cfirst + 1 && want != unit_records[{cons.b, head}]) {
              info[0] = cons.b; info[1] = head; return 10;
            }
          }
        }
        wk.advance(cons);
      }
      if (next != inflight.size()) { info[0] = cta; info[1] = warp; return 11; }
    }
  }
  long long n_direct = 0, n_merged = 0;
  for (int b = 0; b < B; ++b) {
    const int len = seq_lens ? lens[b] : n_seq;
    const int tc = fd_tiles(len, tile);
    for (int h = 0; h < Hkv; ++h) {
      auto it = visited.find({b, h});
      if (it == visited.end() || (int)it->second.size() != tc) { info[0] = b; info[1] = h; return 12; }
      for (int j = 0; j < tc; ++j)
        if (it->second[j] != 1) { info[0] = b; info[1] = h; info[2] = j; info[3] = it->second[j]; return 13; }
      const int d = direct.count({b, h}) ? direct[{b, h}] : 0;
      const int a = arrivals.count({b, h}) ? arrivals[{b, h}] : 0;
      if (d == 1 && a == 0) ++n_direct;
      else if (d == 0 && a >= 2 && a == expected[{b, h}]) ++n_merged;
      else { info[0] = b; info[1] = h; info[2] = d; info[3] = a; return 14; }
    }
  }
  stats[0] = n_direct;
  stats[1] = n_merged;
  stats[2] = n_records;
  return 0;
}

}  // extern "C"
