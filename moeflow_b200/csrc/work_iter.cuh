// How the persistent CTAs of the grouped GEMMs share the work.
//
// A unit is (token tile, 128-row weight block); it needs k_blocks K steps.  The plan word of a GEMM says how
// the units are cut along K:
//   * K split S in {1, 2, 4, 8}: every unit is cut into S equal segments, dealt to the CTAs round-robin;
//   * stream-K (plan word 0): the units' K steps are laid end to end and every CTA takes one contiguous share
//     of that line, so all CTAs stream the same number of weight bytes whatever the unit count; a unit that
//     straddles CTA boundaries is cut there.
// Every warp role of a CTA builds its own iterator from the same plan words and walks the same sequence of
// segments, so the roles stay in step without talking to each other.
#pragma once

#include "common.cuh"
#include "moeflow_b200.h"

namespace mf {

// One piece of work of a CTA: `nkb` K steps of unit (tt, mb) starting at K block kb0.
struct Seg {
  int unit, tt, mb;
  int e, row_start, n_rows;  // the token tile: expert, first entry, entries
  int kb0, nkb;
  int nseg, seg;             // segments of this unit and this one's index in K order (nseg == 1: whole unit)
  int c_first;               // stream-K: CTA that holds segment 0 of the unit
};

// Enumerates the segments of CTA `cta`.  Every warp role builds its own iterator from the same plan words
// and therefore walks the same sequence.
struct WorkIter {
  const mf_gemm_args* a;
  int n_max, m_blocks, KB, split, stream;
  int units;         // n_tiles * m_blocks
  int cta, G;        // this CTA, CTAs that take part
  long long W;       // stream-K: units * KB
  long long w, w1;   // stream-K: cursor and end of this CTA's share
  int u;             // K split: next (unit, split) index
  bool bad_tile;     // a tile wider than the kernel's token tile was met (and skipped)

  __device__ __forceinline__ long long share_begin(int c) const { return (long long)c * W / G; }
  // CTA holding K step x of the line (the largest c with share_begin(c) <= x)
  __device__ __forceinline__ int cta_of(long long x) const { return (int)(((x + 1) * G + W - 1) / W) - 1; }

  __device__ __forceinline__ void init(const mf_gemm_args& args, int n_max_, int n_tiles, int split_, int cta_, int grid) {
    a = &args;
    n_max = n_max_;
    m_blocks = args.m_blocks;
    KB = args.k_blocks;
    split = split_ < 1 ? 1 : split_;
    stream = split_ == 0;
    units = n_tiles * m_blocks;
    cta = cta_;
    W = (long long)units * KB;
    G = stream ? (int)(W < (long long)grid ? W : (long long)grid) : grid;
    bad_tile = false;
    u = cta;
    w = w1 = 0;
    if (stream && cta < G) {
      w = share_begin(cta);
      w1 = share_begin(cta + 1);
    }
  }

  __device__ __forceinline__ bool next(Seg& s) {
    while (true) {
      if (stream) {
        if (w >= w1) return false;
        s.unit = (int)(w / KB);
        s.kb0 = (int)(w - (long long)s.unit * KB);
        const long long left = w1 - w;
        s.nkb = (KB - s.kb0) < left ? (KB - s.kb0) : (int)left;
        w += s.nkb;
        const long long x0 = (long long)s.unit * KB;
        s.c_first = cta_of(x0);
        s.nseg = cta_of(x0 + KB - 1) - s.c_first + 1;
        s.seg = cta - s.c_first;
      } else {
        if (u >= units * split) return false;
        const int ks = u % split;
        s.unit = u / split;
        u += G;
        s.nkb = KB / split;
        s.kb0 = ks * s.nkb;
        s.nseg = split;
        s.seg = ks;
        s.c_first = 0;
      }
      s.tt = s.unit / m_blocks;
      s.mb = s.unit - s.tt * m_blocks;
      s.e = __ldcg(a->tile_e + s.tt);
      s.row_start = __ldcg(a->tile_s + s.tt);
      s.n_rows = __ldcg(a->tile_n + s.tt);
      if ((unsigned)s.n_rows <= (unsigned)n_max) return true;
      bad_tile = true;  // a plan built for wider tiles than this kernel: skip the segment, every role alike
    }
  }

  // Partial-sum slot of segment `sg` of the unit of `s`.  K split: slots are (unit, segment).  Stream-K: every
  // CTA owns two slots, one for the segment its share starts with and one for the segment it ends with.
  __device__ __forceinline__ int slot_of(const Seg& s, int sg) const {
    if (!stream) return s.unit * split + sg;
    const int c = s.c_first + sg;
    return 2 * c + (share_begin(c) >= (long long)s.unit * KB ? 0 : 1);
  }
  // Slots the plan needs (for the capacity check).
  __device__ __forceinline__ long long slots_needed() const {
    if (stream) return 2ll * G;
    return split > 1 ? (long long)units * split : 0;
  }
};

}  // namespace mf
