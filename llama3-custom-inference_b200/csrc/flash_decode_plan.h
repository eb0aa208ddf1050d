// Work partition of the flash-decode kernel, as plain integer functions usable from device code,
// from the host launcher and from a C++ unit test compiled without CUDA.
//
// Vocabulary: a TILE is kTile consecutive cached tokens of one KV head; a COLUMN is the same tile
// for the HG neighbouring KV heads of one head group; a UNIT is one (sequence, KV head) pair, i.e.
// all tiles whose partial results must be merged.  Columns are numbered sequence-major, then head
// group, then tile, and the numbered list is cut into `ctas` contiguous ranges whose sizes differ
// by at most one.  (The reference cuts every sequence into fixed 64-token steps, one CTA each:
// custom_kernels/custom_kernels.cu:243,251,256-259.)
#pragma once

#if defined(__CUDACC__)
#define L3CI_HD __host__ __device__ __forceinline__
#else
#define L3CI_HD inline
#endif

namespace l3ci {

// Tokens per tile: one stage holds a K and a V tile of 4 KiB each.
L3CI_HD constexpr int fd_tile_tokens(int head_size) { return head_size == 128 ? 16 : 32; }

// Warps per CTA = KV heads walked side by side = gcd(Hkv, 8).
L3CI_HD constexpr int fd_head_group(int kv_heads) {
  int a = kv_heads, b = 8;
  while (b) {
    const int t = a % b;
    a = b;
    b = t;
  }
  return a;
}

// Largest useful persistent grid: 8 warps' worth of pipelines fit in one SM's shared memory.
L3CI_HD constexpr int fd_max_ctas(int sms, int head_group) { return sms * (8 / head_group); }

// Tiles of a sequence; an empty sequence still owns one (fully masked) tile so that its output
// rows get written.
L3CI_HD constexpr int fd_tiles(int len, int tile) { return len <= 0 ? 1 : (len + tile - 1) / tile; }

// CTAs that take part when `total` columns meet a grid of `grid` CTAs: never more CTAs than columns,
// so that every participating CTA owns at least one column.
L3CI_HD constexpr int fd_active_ctas(int grid, int total) { return grid < total ? grid : total; }

// First column of CTA `cta` when `total` columns are dealt to `ctas` CTAs.
L3CI_HD constexpr int fd_range_begin(int cta, int total, int ctas) {
  return (int)(((long long)cta * total) / ctas);
}

// The CTA whose range holds column `col`: the largest c with fd_range_begin(c) <= col.
L3CI_HD constexpr int fd_cta_of(int col, int total, int ctas) {
  return (int)((((long long)col + 1) * ctas - 1) / total);
}

// Whole-unit cut.  When sequences are short, cutting them across CTAs buys little streaming time and costs a
// cross-CTA merge (several dependent memory round trips).  The alternative gives every CTA whole
// (sequence, head group) units: units u of CTA c are [c * units / ctas, (c + 1) * units / ctas), ctas =
// min(grid, units).  The choice compares rough costs in units of ~0.16 us: a column costs a CTA of a busy device
// about 9 and of a part-filled device about 6, the merge tail about 38.  It depends on launch-wide numbers only,
// so every CTA decides alike.  (Measured on B200 with 64 sequences, 8 KV heads of 64: whole units take
// 6.3 us + 0.9 us per column of a unit, the cut 12.3 us + 1.45 us per column of a CTA; they cross near 700
// tokens.)
L3CI_HD constexpr bool fd_whole_units(int total, int units, int grid) {
  if (units <= 0 || total <= 0) return false;
  const int ga = grid < units ? grid : units;
  const int gs = grid < total ? grid : total;
  const long long whole = (long long)((units + ga - 1) / ga) * ((total + units - 1) / units) * 6;
  const long long split = (long long)((total + gs - 1) / gs) * 9 + 38;
  return whole < split;
}

// Scratch record written by warp `warp` of CTA `cta` for a unit whose first column lies in CTA
// `first_cta`.  A CTA leaves at most two records per warp: slot 0 for a unit that began in an
// earlier CTA, slot 1 for a unit that begins here and runs on into the next CTA.
L3CI_HD constexpr int fd_record_index(int cta, int first_cta, int head_group, int warp) {
  return (cta * 2 + (cta == first_cta ? 1 : 0)) * head_group + warp;
}


// ---------------------------------------------------------------------------------------------
// Walk over the columns of a CTA's range: (sequence b, head group g, tile j).
// ---------------------------------------------------------------------------------------------
struct FdCursor {
  int col;   // global column index
  int b, g, j;
  int tc;    // tiles of sequence b
  int len;   // valid tokens of sequence b
};

struct FdWalker {
  const int* pref;  // pref[b] = columns before sequence b, pref[B] = total; null when every sequence
                    // has n_seq tokens
  const int* lens;  // clamped lengths; null together with pref
  int B, n_groups, n_seq, tile;

  L3CI_HD int len_of(int b) const { return lens ? lens[b] : n_seq; }
  L3CI_HD int pref_of(int b) const { return pref ? pref[b] : b * n_groups * fd_tiles(n_seq, tile); }
  L3CI_HD int total() const { return pref_of(B); }

  L3CI_HD FdCursor seek(int col) const {
    FdCursor c;
    c.col = col;
    if (pref) {
      int lo = 0, hi = B;  // largest b in [0, B) with pref[b] <= col
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pref[mid] <= col) lo = mid; else hi = mid;
      }
      c.b = lo;
    } else {
      c.b = col / (n_groups * fd_tiles(n_seq, tile));
    }
    c.len = len_of(c.b);
    c.tc = fd_tiles(c.len, tile);
    const int local = col - pref_of(c.b);
    c.g = local / c.tc;
    c.j = local - c.g * c.tc;
    return c;
  }

  L3CI_HD void advance(FdCursor& c) const {
    ++c.col;
    if (++c.j == c.tc) {
      c.j = 0;
      if (++c.g == n_groups) {
        c.g = 0;
        if (++c.b < B) {
          c.len = len_of(c.b);
          c.tc = fd_tiles(c.len, tile);
        }
      }
    }
  }

  // First column of the unit the cursor is in, and the CTAs that unit spans.
  L3CI_HD int unit_begin(const FdCursor& c) const { return pref_of(c.b) + c.g * c.tc; }
};

// ---------------------------------------------------------------------------------------------
// Static deal (flash_decode_small.cu): units handed to warps, CTAs or clusters on the host.
// ---------------------------------------------------------------------------------------------
constexpr int kFdStaticWarps = 8;  // warps of a CTA of the static kernel

// W warps per unit, C CTAs per unit, and the resulting grid; ctas == 0: no split keeps the grid within one wave.
struct FdStaticSplit {
  int W, C, ctas;
};

// The split for `units` units of `tiles` tiles on `sms` SMs.  Few units of at least 32 tiles are spread over
// clusters while every warp still gets a tile and all clusters run at once (max_clusters[i]: clusters of 2 << i
// CTAs the device holds at once); more units than SMs share CTAs.
inline FdStaticSplit fd_static_split(long long units, long long tiles, int sms, const int max_clusters[3]) {
  FdStaticSplit s{kFdStaticWarps, 1, 0};
  if (units <= 0 || sms <= 0) return s;
  if (units <= sms) {
    for (int i = 0; i < 3; ++i) {
      const int c2 = s.C * 2;
      if (tiles < 32 || tiles < (long long)kFdStaticWarps * c2 || units * c2 > sms || units > max_clusters[i]) break;
      s.C = c2;
    }
    s.ctas = (int)(units * s.C);
    return s;
  }
  for (int U = 2; U <= kFdStaticWarps; U *= 2)
    if ((units + U - 1) / U <= sms) {
      s.W = kFdStaticWarps / U;
      s.ctas = (int)((units + U - 1) / U);
      return s;
    }
  return s;
}

// Clusters whose CTAs each get a long run of tiles (384 or more) take the shape with 12 warps and 2 tiles in flight
// per warp instead of 8 and 3.
inline bool fd_static_wide(const FdStaticSplit& s, long long tiles) { return s.C > 1 && tiles / s.C >= 384; }

// Whether a call goes to the static kernel, from host-side sizes only.  Fits to measurements on a B200, bytes per
// microsecond: the static kernel starts in about 4 us, an SM takes in up to 96e3 (256-byte rows, head size 128) or
// 73e3 (128-byte rows, head size 64), 105e3 / 100e3 in the 12-warp shape, all SMs together 6.5e6; the persistent
// kernel, when large, takes 14.8 us plus the bytes at 7.3e6.  Shares (bytes of cache per CTA, from the cache
// length) up to 1 MB always go static, up to 9 MB if the estimates say so; with device-side lengths (ragged)
// the share is held to 1.25 MB, because one long sequence among short ones would keep a single CTA busy.
inline bool fd_static_applies(const FdStaticSplit& s, long long units, long long tiles, int head_size, int n_seq, int ratio,
                              bool ragged) {
  if (ratio > 8 || s.ctas == 0) return false;
  const double unit_bytes = (double)n_seq * 4.0 * head_size;
  const double cta_bytes = unit_bytes * (kFdStaticWarps / s.W) / s.C;
  if (cta_bytes > (ragged ? 1.25e6 : 9.0e6)) return false;
  if (cta_bytes <= 1.0e6) return true;
  const double all = 6.5e6 / s.ctas;
  const double one = fd_static_wide(s, tiles) ? (head_size == 64 ? 100e3 : 105e3) : (head_size == 64 ? 73e3 : 96e3);
  const double t_static = 4.0 + cta_bytes / (one < all ? one : all);
  const double t_persistent = 14.8 + unit_bytes * (double)units / 7.3e6;
  return t_static <= t_persistent;
}

// True when the cursor stands on the last column its CTA sees of the current unit.
L3CI_HD bool fd_unit_ends(const FdCursor& c, int range_end) { return c.j == c.tc - 1 || c.col == range_end - 1; }

}  // namespace l3ci
