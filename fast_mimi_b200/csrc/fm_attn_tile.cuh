// Per-thread pieces of the banded-attention softmax that the whole-clip and the long-clip kernels share:
// one query row per thread, a 128 x 128 FP32 score tile in tensor memory, the causal window
// (key j visible to query i iff max(i - window + 1, 0) <= j <= i; src/fast_mimi/model.py:1672-1676).
#pragma once

#include "fm_common.cuh"

namespace fm {
namespace attn_tile {
constexpr int kTile = 128;
constexpr int kD = 64;

// Which 32-column groups of a 128 x 128 score tile matter to a warp whose rows are frames
// w_row0 .. w_row0+31, against keys k0 .. k0+127, under the causal window.
struct GroupVis {
  int vis_lo, vis_hi;   // this thread's visible columns
  int any_lo, any_hi;   // columns seen by at least one row of the warp
  int all_lo, all_hi;   // columns seen by every row of the warp
  __device__ __forceinline__ GroupVis(int i, int w_row0, int k0, int window)
      : vis_lo(first_key(i, window) - k0), vis_hi(i - k0), any_lo(first_key(w_row0, window) - k0),
        any_hi(w_row0 + 31 - k0), all_lo(first_key(w_row0 + 31, window) - k0), all_hi(w_row0 - k0) {}
  // oldest key frame query i may see; never before the clip's first frame (k0 can be negative for a tile
  // that lies partly or wholly before the clip)
  static __device__ __forceinline__ int first_key(int i, int window) { return i - window + 1 > 0 ? i - window + 1 : 0; }
  __device__ __forceinline__ bool skip(int c0) const { return c0 > any_hi || c0 + 31 < any_lo; }
  __device__ __forceinline__ bool full(int c0) const { return c0 >= all_lo && c0 + 31 <= all_hi; }
};

// Row maximum of the visible raw scores of a tile (this thread's row).
__device__ __forceinline__ float tile_row_max(uint32_t s_addr, const GroupVis& g) {
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    if (g.skip(c0)) continue;
    uint32_t s[32];
    tmem_ld32(s_addr + c0, s);
    tmem_ld_wait();
    if (g.full(c0)) {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    } else {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc)
        if (c0 + cc >= g.vis_lo && c0 + cc <= g.vis_hi) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    }
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// exp2(scale * s - m) of this thread's tile row, written over the consumed scores as packed 16-bit pairs
// (32 keys -> 16 columns, ascending, so a group's P never lands on scores that are still to be read).
// Returns the row sum.
template <typename VT>
__device__ __forceinline__ float tile_row_probs(uint32_t s_addr, uint32_t p_addr, const GroupVis& g, float scale_log2e,
                                                float m_use) {
  float l[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    uint32_t pk[16];
    if (g.skip(c0)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) pk[j] = 0u;
    } else {
      uint32_t s[32];
      tmem_ld32(s_addr + c0, s);
      tmem_ld_wait();
      if (g.full(c0)) {
#pragma unroll
        for (int cc = 0; cc < 32; cc += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(s[cc]), scale_log2e, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(s[cc + 1]), scale_log2e, -m_use));
          pk[cc / 2] = Pack16<VT>::pack(p0, p1);
          l[(cc >> 1) & 3] += p0 + p1;
        }
      } else {
#pragma unroll
        for (int cc = 0; cc < 32; cc += 2) {
          float p[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool vis = c0 + cc + e >= g.vis_lo && c0 + cc + e <= g.vis_hi;
            p[e] = vis ? ex2_approx(fmaf(__uint_as_float(s[cc + e]), scale_log2e, -m_use)) : 0.f;
          }
          pk[cc / 2] = Pack16<VT>::pack(p[0], p[1]);
          l[(cc >> 1) & 3] += p[0] + p[1];
        }
      }
    }
    tmem_st16(p_addr + (c0 >> 1), pk);
  }
  tmem_st_wait();
  return (l[0] + l[1]) + (l[2] + l[3]);
}

// Softmax numerators of this thread's tile row in ONE pass over tensor memory, in place (P over the consumed
// scores as in tile_row_probs).  Softmax is invariant under the offset that is subtracted before exponentiating, so
// the offset need not be the row maximum: it is the (scaled) maximum of the row's first visible 32-key group, and a
// later group is exponentiated against it WITHOUT waiting for that group's own maximum, which is reduced beside the
// exponentials on the integer pipe and only checked afterwards.  If it exceeds the offset by more than kOnlineSlack
// (P would approach the top of the 16-bit range), the warp takes a detour: the offset is raised by a whole number of
// powers of two, the probabilities already written and the running sum are scaled down by that power (exact for
// 16-bit floats short of underflow), and the group, whose scores are still in registers, is redone.  Returns the row
// sum; `offset` is the final offset in log2 units (-inf: no visible key, row sum 0) - whoever combines partial
// results uses it as they would use a maximum.
constexpr float kOnlineSlack = 13.f;       // P < 2^13 without a detour; FP16 holds 2^16, BF16 far more
template <typename VT>
__device__ __forceinline__ float tile_row_softmax_online(uint32_t s_addr, const GroupVis& g, float scale_log2e, float& offset) {
  float l[4] = {0.f, 0.f, 0.f, 0.f};
  float m_off = -INFINITY;
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    uint32_t pk[16];
    if (g.skip(c0)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) pk[j] = 0u;
      tmem_st16(s_addr + (c0 >> 1), pk);
      continue;
    }
    uint32_t s[32];
    tmem_ld32(s_addr + c0, s);
    tmem_ld_wait();
    const bool full = g.full(c0);
    float gm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (full) {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc) gm[cc & 3] = fmaxf(gm[cc & 3], __uint_as_float(s[cc]));
    } else {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc)
        if (c0 + cc >= g.vis_lo && c0 + cc <= g.vis_hi) gm[cc & 3] = fmaxf(gm[cc & 3], __uint_as_float(s[cc]));
    }
    const float gmax = fmaxf(fmaxf(gm[0], gm[1]), fmaxf(gm[2], gm[3])) * scale_log2e;   // -inf: nothing visible here
    // Rows that have not seen a key yet take this group's maximum as their offset (the only place where the
    // exponentials wait for a reduction).
    if (__any_sync(0xffffffffu, m_off == -INFINITY)) {
      if (m_off == -INFINITY) m_off = gmax;
    }
    float lt[4];
    auto exponentiate = [&](float m_use) {
      lt[0] = lt[1] = lt[2] = lt[3] = 0.f;
      if (full) {
#pragma unroll
        for (int cc = 0; cc < 32; cc += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(s[cc]), scale_log2e, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(s[cc + 1]), scale_log2e, -m_use));
          pk[cc / 2] = Pack16<VT>::pack(p0, p1);
          lt[(cc >> 1) & 3] += p0 + p1;
        }
      } else {
#pragma unroll
        for (int cc = 0; cc < 32; cc += 2) {
          float p[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool vis = c0 + cc + e >= g.vis_lo && c0 + cc + e <= g.vis_hi;
            p[e] = vis ? ex2_approx(fmaf(__uint_as_float(s[cc + e]), scale_log2e, -m_use)) : 0.f;
          }
          pk[cc / 2] = Pack16<VT>::pack(p[0], p[1]);
          lt[(cc >> 1) & 3] += p[0] + p[1];
        }
      }
    };
    exponentiate((m_off == -INFINITY) ? 0.f : m_off);
    const bool over = gmax > m_off + kOnlineSlack;         // false while m_off or gmax is -inf
    if (__any_sync(0xffffffffu, over)) {
      // warp-collective detour (rare): raise the offset, scale what the row has accumulated, redo this group
      float down = 1.f;
      if (over) {
        const float k = ceilf(gmax - m_off);
        down = ex2_approx(-k);                             // an exact power of two
        m_off += k;
      }
#pragma unroll 1
      for (int p0 = 0; p0 < (c0 >> 1); p0 += 16) {
        uint32_t w[16];
        tmem_ld16(s_addr + p0, w);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 f = Pack16<VT>::unpack(w[j]);
          w[j] = Pack16<VT>::pack(f.x * down, f.y * down);
        }
        tmem_st16(s_addr + p0, w);
      }
      tmem_st_wait();
#pragma unroll
      for (int j = 0; j < 4; ++j) l[j] *= down;
      exponentiate((m_off == -INFINITY) ? 0.f : m_off);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) l[j] += lt[j];
    tmem_st16(s_addr + (c0 >> 1), pk);
  }
  tmem_st_wait();
  offset = m_off;
  return (l[0] + l[1]) + (l[2] + l[3]);
}

// This thread's 64 output values from TMEM, normalised, rounded, into row `lane` of a swizzled slab.
template <typename VT>
__device__ __forceinline__ void stage_output_row(uint32_t o_addr, uint8_t* slab, int lane, float inv) {
#pragma unroll
  for (int d0 = 0; d0 < kD; d0 += 32) {
    uint32_t o[32];
    tmem_ld32(o_addr + d0, o);
    tmem_ld_wait();
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = Pack16<VT>::pack(__uint_as_float(o[8 * cc + 2 * e]) * inv, __uint_as_float(o[8 * cc + 2 * e + 1]) * inv);
      *reinterpret_cast<uint4*>(slab + sw128_offset(lane, d0 / 8 + cc)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}
// Same for a row whose result is the weighted sum of two partial outputs:  c_a * O_a + c_b * O_b.
template <typename VT>
__device__ __forceinline__ void stage_output_row2(uint32_t oa_addr, uint32_t ob_addr, uint8_t* slab, int lane, float c_a,
                                                  float c_b) {
#pragma unroll
  for (int d0 = 0; d0 < kD; d0 += 32) {
    uint32_t oa[32], ob[32];
    tmem_ld32(oa_addr + d0, oa);
    tmem_ld32(ob_addr + d0, ob);
    tmem_ld_wait();
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = 8 * cc + 2 * e;
        w[e] = Pack16<VT>::pack(fmaf(__uint_as_float(oa[j]), c_a, __uint_as_float(ob[j]) * c_b),
                                fmaf(__uint_as_float(oa[j + 1]), c_a, __uint_as_float(ob[j + 1]) * c_b));
      }
      *reinterpret_cast<uint4*>(slab + sw128_offset(lane, d0 / 8 + cc)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}
// This thread's 64 output values from TMEM, normalised, rounded, straight to its frame's 128 bytes in global
// memory (`dst` null: the loads still run, they are warp-collective, but nothing is stored).
template <typename VT>
__device__ __forceinline__ void store_output_row(uint32_t o_addr, uint16_t* dst, float inv) {
#pragma unroll
  for (int d0 = 0; d0 < kD; d0 += 32) {
    uint32_t o[32];
    tmem_ld32(o_addr + d0, o);
    tmem_ld_wait();
    if (dst != nullptr) {
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          w[e] = Pack16<VT>::pack(__uint_as_float(o[8 * cc + 2 * e]) * inv, __uint_as_float(o[8 * cc + 2 * e + 1]) * inv);
        reinterpret_cast<uint4*>(dst + d0)[cc] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}
// Same for the weighted sum of two partial outputs:  c_a * O_a + c_b * O_b.
template <typename VT>
__device__ __forceinline__ void store_output_row2(uint32_t oa_addr, uint32_t ob_addr, uint16_t* dst, float c_a, float c_b) {
#pragma unroll
  for (int d0 = 0; d0 < kD; d0 += 32) {
    uint32_t oa[32], ob[32];
    tmem_ld32(oa_addr + d0, oa);
    tmem_ld32(ob_addr + d0, ob);
    tmem_ld_wait();
    if (dst != nullptr) {
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 8 * cc + 2 * e;
          w[e] = Pack16<VT>::pack(fmaf(__uint_as_float(oa[j]), c_a, __uint_as_float(ob[j]) * c_b),
                                  fmaf(__uint_as_float(oa[j + 1]), c_a, __uint_as_float(ob[j + 1]) * c_b));
        }
        reinterpret_cast<uint4*>(dst + d0)[cc] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}
}  // namespace attn_tile
}  // namespace fm
