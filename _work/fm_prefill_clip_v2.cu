// Banded causal attention for whole clips of 128 < T <= 256 frames (Mimi's 10 s clips: T = 250), sm_100a.
// Same contract as the general prefill kernel (fm_prefill.cu): rotated q, k (BF16) and v (16-bit) in
// [B, T, 512], output [B, T, 512]; replaces the masked SDPA call of the reference
// (src/fast_mimi/model.py:1860-1868 with the band of src/fast_mimi/model.py:1672-1676).
//
// A persistent CTA takes (clip, head) items.  All of an item's operands — Q, K, V for both 128-frame
// halves, 96 KB — arrive in one TMA batch, and the next item's batch is in flight while the current one
// is computed (two 96 KB buffers).  The three score tiles of the causal band
//     S00 = rows 0-127 x keys 0-127,  S10 = rows 128-255 x keys 0-127,  S11 = rows 128-255 x keys 128-255
// are issued back to back into 384 TMEM columns, so a softmax row sees all of its scores at once: one
// pass for the row maximum, one for the probabilities, no running rescale, and the tensor core
// accumulates P V for both key tiles directly in TMEM (2 x 64 columns).
//
// Twelve softmax warps, three per SM sub-partition, each owning one tile:
//     warps 0-3   S00   (frames permuted so that warp w holds frames 96-32w .. 127-32w)
//     warps 4-7   S10   (rows 128-255, keys 0-127; also normalise, stage and store the rows' output)
//     warps 8-11  S11   (rows 128-255, keys 128-255)
// The causal diagonal gives warp w of S00 4-w visible 32-key groups and warp w of S11 w+1, so every
// sub-partition handles nine groups.  The S10 / S11 warps of a row exchange their partial maximum and
// sum through shared memory (named barriers).  P tiles overwrite the item's dead Q / K tiles (plus one
// extra 32 KB tile for P11); outputs are staged in tiles that are dead by then and leave through TMA
// stores.  Warp 12: TMA loads + MMA issue.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace clip {
constexpr int kTile = 128;
constexpr int kD = 64;
constexpr int kTileBytes = kTile * kD * 2;          // 16 KB
constexpr int kSlabBytes = 32 * 128;                // 32 rows x 64 x 16 bit
constexpr int kItemBytes = 6 * kTileBytes;          // Q0 Q1 K0 K1 V0 V1
constexpr int kSoftmaxWarps = 12;
constexpr int kThreads = (kSoftmaxWarps + 1) * 32;
constexpr int kTmemCols = 512;                      // S00 | S10 | S11 | O0 | O1
constexpr uint32_t kS00 = 0, kS10 = 128, kS11 = 256, kO0 = 384, kO1 = 448;

struct Shared {
  uint64_t load_full[2];
  uint64_t buf_free[2];    // the P V products that read a buffer have completed
  uint64_t out_done[2];    // the output staged in a buffer has been read by its TMA stores
  uint64_t s_full[2];      // [0]: S00; [1]: S10 and S11
  uint64_t p_full[2];      // [0]: P00 written (4 warps); [1]: P10 and P11 written (8 warps)
  uint64_t o_full[2];
  uint32_t tmem_base;
  CtaCtl ctl;
  float xm[kTile][2];      // partial row maxima of S10 / S11
  float xl[kTile];         // partial row sums of S11
};
constexpr int kSmemBytes = 1024 + 2 * kItemBytes + 2 * kTileBytes + static_cast<int>((sizeof(Shared) + 127) & ~size_t(127));
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");

// Row maximum of the visible raw scores of one 128 x 128 tile (this thread's row).
__device__ __forceinline__ float tile_row_max(uint32_t s_addr, int i, int w_row0, int k0, int window) {
  const int vis_lo = i - window + 1 - k0, vis_hi = i - k0;
  const int any_lo = w_row0 - window + 1 - k0, any_hi = w_row0 + 31 - k0;   // seen by at least one row of the warp
  const int all_lo = w_row0 + 31 - window + 1 - k0, all_hi = w_row0 - k0;   // seen by every row of the warp
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    if (c0 > any_hi || c0 + 31 < any_lo) continue;
    uint32_t s[32];
    tmem_ld32(s_addr + c0, s);
    tmem_ld_wait();
    if (c0 >= all_lo && c0 + 31 <= all_hi) {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    } else {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc)
        if (c0 + cc >= vis_lo && c0 + cc <= vis_hi) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    }
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// exp2(scale * s - m) of one tile row -> 16-bit P tile (two swizzled 64-key halves); returns the row sum.
template <typename VT>
__device__ __forceinline__ float tile_row_probs(uint32_t s_addr, uint8_t* p_lo, uint8_t* p_hi, int r, int i, int w_row0,
                                                int k0, int window, float scale_log2e, float m_use) {
  const int vis_lo = i - window + 1 - k0, vis_hi = i - k0;
  const int any_lo = w_row0 - window + 1 - k0, any_hi = w_row0 + 31 - k0;
  const int all_lo = w_row0 + 31 - window + 1 - k0, all_hi = w_row0 - k0;
  float l[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 32) {
    uint8_t* half_base = (c0 >> 6) == 0 ? p_lo : p_hi;
    const int chunk0 = (c0 & 63) >> 3;
    if (c0 > any_hi || c0 + 31 < any_lo) {
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
        *reinterpret_cast<uint4*>(half_base + sw128_offset(r, chunk0 + cc)) = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    uint32_t s[32];
    tmem_ld32(s_addr + c0, s);
    tmem_ld_wait();
    uint32_t pk[16];
    if (c0 >= all_lo && c0 + 31 <= all_hi) {
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
          const bool vis = c0 + cc + e >= vis_lo && c0 + cc + e <= vis_hi;
          p[e] = vis ? ex2_approx(fmaf(__uint_as_float(s[cc + e]), scale_log2e, -m_use)) : 0.f;
        }
        pk[cc / 2] = Pack16<VT>::pack(p[0], p[1]);
        l[(cc >> 1) & 3] += p[0] + p[1];
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc)
      *reinterpret_cast<uint4*>(half_base + sw128_offset(r, chunk0 + cc)) =
          make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
  }
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

__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
}  // namespace clip

template <typename VT>
__global__ void __launch_bounds__(clip::kThreads, 1)
band_attn_clip_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_q32,
                      const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ CUtensorMap tmap_out, int n_items, int T, int window,
                      float scale_log2e, int* status) {
  using namespace clip;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_p11 = smem + 2 * kItemBytes;
  Shared* sh = reinterpret_cast<Shared*>(smem_p11 + 2 * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->load_full[i], 1);
      mbar_init(&sh->buf_free[i], 1);
      mbar_init(&sh->out_done[i], 8);
      mbar_init(&sh->s_full[i], 1);
      mbar_init(&sh->o_full[i], 1);
    }
    mbar_init(&sh->p_full[0], 4);
    mbar_init(&sh->p_full[1], 8);
    sh->ctl.abort = 0;
    fence_mbar_init();
  }
  if (warp == kSoftmaxWarps) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  CtaCtl* ctl = &sh->ctl;
  const int n_local = (n_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  if (warp == kSoftmaxWarps) {
    // ------------------------------------------------------------ TMA loads + MMA issue
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_q32);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      auto load_item = [&](int n) {
        const int item = blockIdx.x + n * gridDim.x;
        const int c = item >> 3, h = item & 7, b = n & 1;
        uint8_t* base = smem + b * kItemBytes;
        mbar_arrive_expect_tx(&sh->load_full[b], kItemBytes);
        // Q0 in four 32-frame boxes, block j of the tile <- frames 96-32j .. 127-32j.
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_load_3d(base + j * kSlabBytes, &tmap_q32, &sh->load_full[b], h * kD, (3 - j) * 32, c);
        tma_load_3d(base + 1 * kTileBytes, &tmap_q, &sh->load_full[b], h * kD, kTile, c);
        tma_load_3d(base + 2 * kTileBytes, &tmap_k, &sh->load_full[b], h * kD, 0, c);
        tma_load_3d(base + 3 * kTileBytes, &tmap_k, &sh->load_full[b], h * kD, kTile, c);
        tma_load_3d(base + 4 * kTileBytes, &tmap_v, &sh->load_full[b], h * kD, 0, c);
        tma_load_3d(base + 5 * kTileBytes, &tmap_v, &sh->load_full[b], h * kD, kTile, c);
      };
      constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kD, Pack16<VT>::kFmt, Pack16<VT>::kFmt, 0, 1);
      if (n_local > 0) load_item(0);
      for (int n = 0; n < n_local; ++n) {
        const int b = n & 1;
        uint8_t* base = smem + b * kItemBytes;
        mbar_wait(&sh->load_full[b], static_cast<uint32_t>(n >> 1) & 1u, ctl, status, kErrWaitTma);
        tc_fence_after_sync();
        const uint64_t q0 = umma_desc_sw128(smem_u32(base)), q1 = umma_desc_sw128(smem_u32(base + kTileBytes));
        const uint64_t k0 = umma_desc_sw128(smem_u32(base + 2 * kTileBytes));
        const uint64_t k1 = umma_desc_sw128(smem_u32(base + 3 * kTileBytes));
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) tc_mma_ss(tmem_base + kS00, q0 + 2u * ks, k0 + 2u * ks, idesc_qk, ks != 0);
        tc_commit(&sh->s_full[0]);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) tc_mma_ss(tmem_base + kS10, q1 + 2u * ks, k0 + 2u * ks, idesc_qk, ks != 0);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) tc_mma_ss(tmem_base + kS11, q1 + 2u * ks, k1 + 2u * ks, idesc_qk, ks != 0);
        tc_commit(&sh->s_full[1]);
        if (n + 1 < n_local) {
          if (n >= 1) {
            // The other buffer held item n-1: its P V reads and its staged output must be finished.
            const uint32_t ph = static_cast<uint32_t>((n - 1) >> 1) & 1u;
            mbar_wait(&sh->buf_free[b ^ 1], ph, ctl, status, kErrWaitMma);
            mbar_wait(&sh->out_done[b ^ 1], ph, ctl, status, kErrWaitConsumer);
          }
          load_item(n + 1);
        }
        const uint64_t v0 = umma_desc_sw128(smem_u32(base + 4 * kTileBytes));
        const uint64_t v1 = umma_desc_sw128(smem_u32(base + 5 * kTileBytes));
        // rows 0-127: O0 = P00 V0 (P00 lives where Q0, Q1 were)
        mbar_wait(&sh->p_full[0], static_cast<uint32_t>(n) & 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) {
          const uint64_t p = umma_desc_sw128(smem_u32(base + (ks >> 2) * kTileBytes)) + 2u * (ks & 3);
          tc_mma_ss(tmem_base + kO0, p, v0 + static_cast<uint64_t>(ks) * 128u, idesc_pv, ks != 0);
        }
        tc_commit(&sh->o_full[0]);
        // rows 128-255: O1 = P10 V0 + P11 V1 (P10 where K0, K1 were; P11 in the extra tile)
        mbar_wait(&sh->p_full[1], static_cast<uint32_t>(n) & 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) {
          const uint64_t p = umma_desc_sw128(smem_u32(base + (2 + (ks >> 2)) * kTileBytes)) + 2u * (ks & 3);
          tc_mma_ss(tmem_base + kO1, p, v0 + static_cast<uint64_t>(ks) * 128u, idesc_pv, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) {
          const uint64_t p = umma_desc_sw128(smem_u32(smem_p11 + (ks >> 2) * kTileBytes)) + 2u * (ks & 3);
          tc_mma_ss(tmem_base + kO1, p, v1 + static_cast<uint64_t>(ks) * 128u, idesc_pv, 1u);
        }
        tc_commit(&sh->o_full[1]);
        tc_commit(&sh->buf_free[b]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int role = warp >> 2;               // 0: S00, 1: S10, 2: S11
    const int lg = warp & 3;                  // TMEM lane group
    const int r = lg * 32 + lane;             // row of the tile == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(lg * 32) << 16;
    // First frame held by this warp, and this thread's frame.
    const int w_row0 = role == 0 ? (3 - lg) * 32 : kTile + lg * 32;
    const int i = w_row0 + lane;
    for (int n = 0; n < n_local; ++n) {
      const int item = blockIdx.x + n * gridDim.x;
      const int c = item >> 3, h = item & 7, b = n & 1;
      const uint32_t ph = static_cast<uint32_t>(n) & 1u;
      uint8_t* base = smem + b * kItemBytes;
      if (role == 0) {
        mbar_wait(&sh->s_full[0], ph, ctl, status, kErrWaitMma);
        tc_fence_after_sync();
        const float m_raw = tile_row_max(tmem_base + lane_sel + kS00, i, w_row0, 0, window);
        const float m_use = (m_raw == -INFINITY) ? 0.f : m_raw * scale_log2e;
        // The second half of P00 overwrites Q1, which S10 / S11 still read until s_full[1].
        mbar_wait(&sh->s_full[1], ph, ctl, status, kErrWaitMma);
        const float l_row = tile_row_probs<VT>(tmem_base + lane_sel + kS00, base, base + kTileBytes, r, i, w_row0, 0,
                                               window, scale_log2e, m_use);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_full[0]);

        mbar_wait(&sh->o_full[0], ph, ctl, status, kErrWaitMma);
        tc_fence_after_sync();
        uint8_t* slab = base + lg * kSlabBytes;                 // inside the dead Q0 tile
        stage_output_row<VT>(tmem_base + lane_sel + kO0, slab, lane, 1.f / l_row);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (w_row0 < T) {                                     // frames past T are clipped by the map
            tma_store_3d(&tmap_out, slab, h * kD, w_row0, c);
            bulk_commit_group();
            bulk_wait_group_read<0>();
          }
          mbar_arrive(&sh->out_done[b]);
        }
      } else if (role == 1) {
        mbar_wait(&sh->s_full[1], ph, ctl, status, kErrWaitMma);
        tc_fence_after_sync();
        const float m_a = tile_row_max(tmem_base + lane_sel + kS10, i, w_row0, 0, window);
        sh->xm[r][0] = m_a;
        named_bar_sync(1 + lg, 64);
        const float m_raw = fmaxf(m_a, sh->xm[r][1]);
        const float m_use = (m_raw == -INFINITY) ? 0.f : m_raw * scale_log2e;
        const float l_a = tile_row_probs<VT>(tmem_base + lane_sel + kS10, base + 2 * kTileBytes, base + 3 * kTileBytes, r,
                                             i, w_row0, 0, window, scale_log2e, m_use);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        // The S11 warp's row sums are read before this warp's arrival lets the next item start, so the
        // next item's sums cannot overwrite them first.
        named_bar_sync(5 + lg, 64);
        const float l_row = l_a + sh->xl[r];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_full[1]);

        mbar_wait(&sh->o_full[1], ph, ctl, status, kErrWaitMma);
        tc_fence_after_sync();
        uint8_t* slab = base + 2 * kTileBytes + lg * kSlabBytes;   // inside the dead K0 tile
        stage_output_row<VT>(tmem_base + lane_sel + kO1, slab, lane, 1.f / l_row);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (w_row0 < T) {
            tma_store_3d(&tmap_out, slab, h * kD, w_row0, c);
            bulk_commit_group();
            bulk_wait_group_read<0>();
          }
          mbar_arrive(&sh->out_done[b]);
        }
      } else {
        mbar_wait(&sh->s_full[1], ph, ctl, status, kErrWaitMma);
        tc_fence_after_sync();
        const float m_b = tile_row_max(tmem_base + lane_sel + kS11, i, w_row0, kTile, window);
        sh->xm[r][1] = m_b;
        named_bar_sync(1 + lg, 64);
        const float m_raw = fmaxf(m_b, sh->xm[r][0]);
        const float m_use = (m_raw == -INFINITY) ? 0.f : m_raw * scale_log2e;
        const float l_b = tile_row_probs<VT>(tmem_base + lane_sel + kS11, smem_p11, smem_p11 + kTileBytes, r, i, w_row0,
                                             kTile, window, scale_log2e, m_use);
        sh->xl[r] = l_b;
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_full[1]);
        named_bar_arrive(5 + lg, 64);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (ctl->abort) __nanosleep(20000);
  if (warp == kSoftmaxWarps) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int encode_clip_map(CUtensorMap* map, const void* base, int B, int T, uint32_t box_rows) {
  // [B, T, 512] 16-bit viewed as (512 fastest, T, B); box = 64 columns x box_rows frames of one clip.
  const cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(T) * 512 * 2};
  const cuuint32_t box[3] = {64, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

int launch_band_attn_clip(const void* q, const void* k, const void* v, void* out, int B, int T, int window, float scale,
                          int value_is_fp16, int* status, cudaStream_t st) {
  using namespace clip;
  if (T <= kTile || T > 2 * kTile || B <= 0 || window <= 0) return -1;
  CUtensorMap tq, tq32, tk, tv, tout;
  int rc = encode_clip_map(&tq, q, B, T, kTile);
  if (rc == 0) rc = encode_clip_map(&tq32, q, B, T, 32);
  if (rc == 0) rc = encode_clip_map(&tk, k, B, T, kTile);
  if (rc == 0) rc = encode_clip_map(&tv, v, B, T, kTile);     // element size is what matters: 16 bit
  if (rc == 0) rc = encode_clip_map(&tout, out, B, T, 32);
  if (rc != 0) return rc;
  auto kern = value_is_fp16 ? band_attn_clip_kernel<__half> : band_attn_clip_kernel<__nv_bfloat16>;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (rc != 0) return rc;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = B * 8;
  const int grid = n_items < sms ? n_items : sms;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tq, tq32, tk, tv, tout, n_items, T, window, scale * 1.4426950408889634f,
                                          status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
