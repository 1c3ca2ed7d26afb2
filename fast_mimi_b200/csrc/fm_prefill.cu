// Banded causal attention (prefill) for sm_100a: H=8 heads of D=64, sliding window W.
//
//   out[b, i, h, :] = softmax_j( scale * q[b,i,h,:] . k[b,j,h,:] ) v[b,j,h,:],  i-W < j <= i
//
// Replaces the masked SDPA call of the reference (src/fast_mimi/model.py:1860-1868, mask
// src/fast_mimi/model.py:1672-1676; functional form src/fast_mimi/_functional_runtime.py:262-269)
// and its native-window variant (src/fast_mimi/model.py:1589-1624).  q and k arrive already rotated.
//
// One CTA owns a 128-query tile of one (clip, head).  Only key tiles that intersect the band
// [q0-W+1, q0+127] are visited (at most three 128-key tiles for W=250, whatever T is).  Q, K and V
// tiles are staged by TMA (128-byte swizzle) from the [B, T, 512] tensors through a 3-D tensor map,
// so frames past the end of a clip read as zero.  S = Q K^T and O_j = P_j V_j run as tcgen05.mma
// with TMEM accumulators; the softmax warps own one query row per thread (tcgen05.ld 32x32b), keep
// the running maximum / sum / output in registers, and hand P_j back through shared memory as a
// K-major swizzled 16-bit tile.  Warps 0-3: softmax + output.  Warp 4: TMA + MMA issue.
//
// The same kernel serves calls whose keys start before their queries (a chunk of new frames attending to
// cached frames plus itself, src/fast_mimi/model.py:2194-2205 with query_offset = past and key_offset =
// max(past - (W-1), 0)): query row i of Tq sits `delta` = query_offset - key_offset rows further along the
// key axis, key row j of Tk = delta + Tq is visible iff  i + delta - W < j <= i + delta.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace fmha {
constexpr int kTile = 128;
constexpr int kD = 64;
constexpr int kTileBytes = kTile * kD * 2;  // 16 KB: 128 rows x 128 B
constexpr int kKvStages = 2;
constexpr int kThreads = 160;
constexpr int kTmemCols = 256;              // S: 128 columns, O: 2 x 64 columns
// P_j (128 x 128 x 16 bit = 32 KB) reuses the K_j stage for its first 64-key half: K_j is dead once
// S_j = Q K_j^T has completed, and the stage is not refilled before P_j V_j has completed.
constexpr int kSmemBytes = 1024 + kTileBytes /*Q*/ + kKvStages * 2 * kTileBytes /*K,V*/ + kTileBytes /*P hi*/ + 256;

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[kKvStages];
  uint64_t kv_empty[kKvStages];
  uint64_t s_full;
  uint64_t p_full;
  uint64_t o_full[2];
  uint64_t o_empty[2];
  uint32_t tmem_base;
  CtaCtl ctl;
};
static_assert(sizeof(Barriers) <= 256, "barrier block too large");
}  // namespace fmha

template <typename VT>
__global__ void __launch_bounds__(fmha::kThreads, 2)
band_attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, uint16_t* __restrict__ out, int T, int Tk,
                         int delta, int window, float scale_log2e, int* status) {
  using namespace fmha;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;
  uint8_t* smem_kv = smem_q + kTileBytes;                     // stage s: K at 2s, V at 2s+1
  uint8_t* smem_p_hi = smem_kv + kKvStages * 2 * kTileBytes;  // keys 64..127 of P_j (keys 0..63 alias K_j)
  Barriers* bars = reinterpret_cast<Barriers*>(smem_p_hi + kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, clip = blockIdx.z;
  const int q0 = qt * kTile;
  const int band_lo = q0 + delta - (window - 1);            // oldest key row any query of the tile may see
  const int j_lo = band_lo > 0 ? band_lo / kTile : 0;       // first key tile touching the band
  const int band_hi = q0 + kTile - 1 + delta < Tk - 1 ? q0 + kTile - 1 + delta : Tk - 1;
  const int j_hi = band_hi / kTile;                         // == qt when keys and queries coincide
  const int n_kv = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kKvStages; ++i) {
      mbar_init(&bars->kv_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_full, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->o_full[i], 1);
      mbar_init(&bars->o_empty[i], 4);
    }
    bars->ctl.abort = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;
  CtaCtl* ctl = &bars->ctl;

  if (warp == 4) {
    // The 32 lanes walk the loop together and one elected lane issues copies, MMAs and commits (warp-uniform
    // control flow keeps the descriptors in uniform registers; a lone lane under a lane test issues slower).
    {
      const bool one = elect_one();
      if (one) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
        mbar_arrive_expect_tx(&bars->q_full, kTileBytes);
        tma_load_3d(smem_q, &tmap_q, &bars->q_full, head * kD, q0, clip);
      }
      auto load_kv = [&](int jj) {
        const int st = jj % kKvStages;
        const uint32_t use = static_cast<uint32_t>(jj / kKvStages);
        mbar_wait(&bars->kv_empty[st], (use & 1u) ^ 1u, ctl, status, kErrWaitConsumer);
        if (one) {
          mbar_arrive_expect_tx(&bars->kv_full[st], 2 * kTileBytes);
          const int k0 = (j_lo + jj) * kTile;
          tma_load_3d(smem_kv + (2 * st) * kTileBytes, &tmap_k, &bars->kv_full[st], head * kD, k0, clip);
          tma_load_3d(smem_kv + (2 * st + 1) * kTileBytes, &tmap_v, &bars->kv_full[st], head * kD, k0, clip);
        }
      };
      for (int jj = 0; jj < n_kv && jj < kKvStages; ++jj) load_kv(jj);

      constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, 1, 1, 0, 0);                       // bf16 x bf16
      constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kD, Pack16<VT>::kFmt, Pack16<VT>::kFmt, 0, 1);  // V is MN-major
      mbar_wait(&bars->q_full, 0, ctl, status, kErrWaitTma);
      const uint64_t q_desc = umma_desc_sw128(smem_u32(smem_q));
      for (int jj = 0; jj < n_kv; ++jj) {
        const int st = jj % kKvStages;
        const uint32_t kv_use = static_cast<uint32_t>(jj / kKvStages);
        mbar_wait(&bars->kv_full[st], kv_use & 1u, ctl, status, kErrWaitTma);
        tc_fence_after_sync();
        const uint64_t k_desc = umma_desc_sw128(smem_u32(smem_kv + (2 * st) * kTileBytes));
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          if (one) tc_mma_ss(tmem_s, q_desc + 2u * ks, k_desc + 2u * ks, idesc_qk, ks != 0 ? 1u : 0u);
        if (one) tc_commit(&bars->s_full);

        // P_j is in shared memory once all four softmax warps have arrived.
        mbar_wait(&bars->p_full, static_cast<uint32_t>(jj) & 1u, ctl, status, kErrWaitConsumer);
        const int ob = jj & 1;
        const uint32_t o_use = static_cast<uint32_t>(jj >> 1);
        mbar_wait(&bars->o_empty[ob], (o_use & 1u) ^ 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        const uint64_t v_desc = umma_desc_sw128(smem_u32(smem_kv + (2 * st + 1) * kTileBytes));
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) {
          // A = P: 64-key halves are separate 16 KB tiles, 32 B per 16-key step inside a half.
          const uint8_t* p_half = (ks >> 2) == 0 ? smem_kv + (2 * st) * kTileBytes : smem_p_hi;
          const uint64_t p_desc = umma_desc_sw128(smem_u32(p_half)) + 2u * (ks & 3);
          // B = V (MN-major): 16 keys = 16 rows of 128 B = 2048 B per step.
          if (one)
            tc_mma_ss(tmem_o + ob * kD, p_desc, v_desc + static_cast<uint64_t>(ks) * (2048u >> 4), idesc_pv,
                      ks != 0 ? 1u : 0u);
        }
        if (one) {
          tc_commit(&bars->o_full[ob]);
          tc_commit(&bars->kv_empty[st]);
        }
        if (jj + kKvStages < n_kv) load_kv(jj + kKvStages);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int r = warp * 32 + lane;          // row inside the tile == TMEM lane
    const int i = q0 + r;                    // query frame
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    float o_acc[kD];
#pragma unroll
    for (int d = 0; d < kD; ++d) o_acc[d] = 0.f;

    for (int jj = 0; jj < n_kv; ++jj) {
      const int k0 = (j_lo + jj) * kTile;
      // A tile needs per-element masking if it crosses the causal diagonal or the window's lower edge.
      const bool need_mask = (k0 + kTile - 1 > q0 + delta) || (k0 < q0 + delta + kTile - window);
      const int vis_lo = i + delta - window + 1 - k0;   // visible columns c: vis_lo <= c <= vis_hi
      const int vis_hi = i + delta - k0;
      mbar_wait(&bars->s_full, static_cast<uint32_t>(jj) & 1u, ctl, status, kErrWaitMma);
      tc_fence_after_sync();

      // A 32-column group is skipped by the whole warp when none of the warp's 32 rows can see it.
      const int warp_vis_lo = q0 + delta + warp * 32 - window + 1 - k0;   // smallest visible column of any row
      const int warp_vis_hi = q0 + delta + warp * 32 + 31 - k0;           // largest
      // Pass 1: row maximum of the visible scores (log2 domain).
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        if (c0 > warp_vis_hi || c0 + 31 < warp_vis_lo) continue;
        uint32_t s[32];
        tmem_ld32(tmem_s + lane_sel + c0, s);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float x = __uint_as_float(s[c]) * scale_log2e;
          if (need_mask && (c0 + c < vis_lo || c0 + c > vis_hi)) x = -INFINITY;
          m_tile = fmaxf(m_tile, x);
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = ex2_approx(m_run - m_use);   // 0 while nothing has been seen yet
      // Pass 2: probabilities -> 16-bit P tile in shared memory, running sum.
      float l_tile = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        uint8_t* half_base = (c0 >> 6) == 0 ? smem_kv + (2 * (jj % kKvStages)) * kTileBytes : smem_p_hi;
        const int chunk0 = (c0 & 63) >> 3;   // first 16-byte chunk (8 keys) of this 32-key group
        if (c0 > warp_vis_hi || c0 + 31 < warp_vis_lo) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
            *reinterpret_cast<uint4*>(half_base + sw128_offset(r, chunk0 + cc)) = make_uint4(0u, 0u, 0u, 0u);
          continue;
        }
        uint32_t s[32];
        tmem_ld32(tmem_s + lane_sel + c0, s);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float p[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float x = __uint_as_float(s[c + e]) * scale_log2e - m_use;
            if (need_mask && (c0 + c + e < vis_lo || c0 + c + e > vis_hi)) x = -INFINITY;
            p[e] = ex2_approx(x);
          }
          pk[c / 2] = Pack16<VT>::pack(p[0], p[1]);
          l_tile += p[0] + p[1];
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          *reinterpret_cast<uint4*>(half_base + sw128_offset(r, chunk0 + cc)) =
              make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      fence_proxy_async_smem();     // P writes -> visible to the tensor core's async proxy
      tc_fence_before_sync();       // orders this thread's S loads before the next S = QK^T
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);

      // O_j = P_j V_j comes back through TMEM; fold it into the register accumulator.
      const int ob = jj & 1;
      mbar_wait(&bars->o_full[ob], static_cast<uint32_t>(jj >> 1) & 1u, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
#pragma unroll
      for (int d0 = 0; d0 < kD; d0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_sel + ob * kD + d0, o);
        tmem_ld_wait();
#pragma unroll
        for (int d = 0; d < 32; ++d) o_acc[d0 + d] = o_acc[d0 + d] * alpha + __uint_as_float(o[d]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_empty[ob]);
    }

    if (i < T) {
      const float inv = 1.f / l_run;
      uint4* dst = reinterpret_cast<uint4*>(out + (static_cast<long long>(clip) * T + i) * 512 + head * kD);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          w[e] = Pack16<VT>::pack(o_acc[8 * c + 2 * e] * inv, o_acc[8 * c + 2 * e + 1] * inv);
        dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (ctl->abort) __nanosleep(20000);
  if (warp == 4) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int encode_clip_tile(CUtensorMap* map, const void* base, int B, int T, CUtensorMapDataType dt) {
  // [B, T, 512] viewed as (512 fastest, T, B); box = 64 columns x 128 frames of one clip.
  const cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(T) * 512 * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_tiled(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int launch_general(const void* q, const void* k, const void* v, void* out, int B, int T, int Tk, int delta,
                          int window, float scale, int value_is_fp16, int* status, cudaStream_t st) {
  using namespace fmha;
  if (B > 65535) return -1;
  CUtensorMap tq, tk, tv;
  int rc = encode_clip_tile(&tq, q, B, T, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (rc != 0) return rc;
  rc = encode_clip_tile(&tk, k, B, Tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (rc != 0) return rc;
  rc = encode_clip_tile(&tv, v, B, Tk, value_is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (rc != 0) return rc;
  auto kern = value_is_fp16 ? band_attn_prefill_kernel<__half> : band_attn_prefill_kernel<__nv_bfloat16>;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (rc != 0) return rc;
  dim3 grid((T + kTile - 1) / kTile, 8, B);
  const float scale_log2e = scale * 1.4426950408889634f;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tq, tk, tv, static_cast<uint16_t*>(out), T, Tk, delta, window, scale_log2e,
                                          status);
  return static_cast<int>(cudaGetLastError());
}

int launch_band_attn_chunk(const void* q, const void* k, const void* v, void* out, int B, int Tq, int Tk, int window,
                           float scale, int value_is_fp16, int* status, cudaStream_t st) {
  if (B <= 0 || Tq <= 0) return (B == 0 || Tq == 0) ? 0 : -1;
  if (window <= 0 || Tk < Tq) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15u)
    return -3;
  if (Tk == Tq) return launch_band_attn_prefill(q, k, v, out, B, Tq, window, scale, value_is_fp16, status, st);
  return launch_general(q, k, v, out, B, Tq, Tk, Tk - Tq, window, scale, value_is_fp16, status, st);
}

int launch_band_attn_prefill(const void* q, const void* k, const void* v, void* out, int B, int T, int window,
                             float scale, int value_is_fp16, int* status, cudaStream_t st) {
  using namespace fmha;
  if (B <= 0 || T <= 0) return (B == 0 || T == 0) ? 0 : -1;
  if (window <= 0 || B > 65535) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15u)
    return -3;
  // Clips that fit two 128-frame tiles take the whole-clip kernel (one CTA per (clip, head) item).
  if (T > kTile && T <= 2 * kTile && B <= (1 << 27))
    return launch_band_attn_clip(q, k, v, out, B, T, window, scale, value_is_fp16, status, st);
  // Longer clips whose window spans exactly three key tiles per query tile take the run-walking kernel.
  if (T > 2 * kTile && window > kTile + 1 && window <= 2 * kTile + 1 && B <= (1 << 27))
    return launch_band_attn_long(q, k, v, out, B, T, window, scale, value_is_fp16, status, st);
  return launch_general(q, k, v, out, B, T, T, 0, window, scale, value_is_fp16, status, st);
}

}  // namespace fm
