// QKV projection with a RoPE epilogue for sm_100a.
//
//   [q | k | v][m, :] = x[m, :] * W_qkv^T          (M frames x 1536 outputs x K=512, BF16 in, FP32 acc)
//   q, k <- rotate-half RoPE at the frame's position  (FP32, before rounding to 16 bit)
//
// Replaces the three bias-free projections plus _apply_rope of the reference
// (src/fast_mimi/model.py:1897-1912; packed form src/fast_mimi/_packed_qkv.py:139-171).
//
// One CTA owns a 128-frame tile of x.  The x tile (128 x 512 BF16 = 128 KB) is loaded once by
// TMA and stays in shared memory; W_qkv streams through a 3-stage ring of 256x64 tiles (it is
// 1.5 MB and lives in L2).  Each 128x256 output tile (4 heads of q, k or v) is accumulated by
// tcgen05.mma into one of two 256-column TMEM buffers, so the epilogue of tile n overlaps the
// MMAs of tile n+1.  Warps 0-3: epilogue (thread = one frame row; both halves of a RoPE pair are
// in that thread's TMEM row).  Warp 4: TMA producer.  Warp 5: MMA issuer.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace gemm {
constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;            // one 128-byte swizzle row of BF16
constexpr int kHidden = 512;           // K
constexpr int kKChunks = kHidden / kBlockK;
constexpr int kStages = 3;
constexpr int kABytes = kBlockM * kBlockK * 2;   // 16 KB per K chunk
constexpr int kBBytes = kBlockN * kBlockK * 2;   // 32 KB per stage
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kSmemBytes = 1024 /*align*/ + kKChunks * kABytes + kStages * kBBytes + 256 /*barriers*/;

struct Barriers {
  uint64_t a_full[kKChunks];
  uint64_t b_full[kStages];
  uint64_t b_empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  CtaCtl ctl;
};
static_assert(sizeof(Barriers) <= 256, "barrier block too large");
}  // namespace gemm

template <typename VT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
qkv_rope_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                     QkvEpilogueArgs ep, int M, int n_tiles_per_cta, int* status) {
  using namespace gemm;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                   // kKChunks x [128 rows x 128 B]
  uint8_t* smem_b = smem + kKChunks * kABytes;              // kStages  x [256 rows x 128 B]
  Barriers* bars = reinterpret_cast<Barriers*>(smem_b + kStages * kBBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kBlockM;
  const int n_first = blockIdx.y * n_tiles_per_cta;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kKChunks; ++i) mbar_init(&bars->a_full[i], 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars->b_full[i], 1);
      mbar_init(&bars->b_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 4);
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
  CtaCtl* ctl = &bars->ctl;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      tma_prefetch_desc(&tmap_w);
      for (int kc = 0; kc < kKChunks; ++kc) {
        mbar_arrive_expect_tx(&bars->a_full[kc], kABytes);
        tma_load_2d(smem_a + kc * kABytes, &tmap_x, &bars->a_full[kc], kc * kBlockK, m0);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int nt = 0; nt < n_tiles_per_cta; ++nt) {
        const int n0 = (n_first + nt) * kBlockN;
        for (int kc = 0; kc < kKChunks; ++kc) {
          mbar_wait(&bars->b_empty[stage], phase ^ 1u, ctl, status, kErrWaitConsumer);
          mbar_arrive_expect_tx(&bars->b_full[stage], kBBytes);
          tma_load_2d(smem_b + stage * kBBytes, &tmap_w, &bars->b_full[stage], kc * kBlockK, n0);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kBlockM, kBlockN, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      for (int nt = 0; nt < n_tiles_per_cta; ++nt) {
        const int buf = nt & 1;
        const uint32_t use = static_cast<uint32_t>(nt >> 1);
        mbar_wait(&bars->acc_empty[buf], (use & 1u) ^ 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kBlockN);
        for (int kc = 0; kc < kKChunks; ++kc) {
          if (nt == 0) mbar_wait(&bars->a_full[kc], 0, ctl, status, kErrWaitTma);
          mbar_wait(&bars->b_full[stage], phase, ctl, status, kErrWaitTma);
          tc_fence_after_sync();
          const uint64_t a_desc = umma_desc_sw128(smem_u32(smem_a + kc * kABytes));
          const uint64_t b_desc = umma_desc_sw128(smem_u32(smem_b + stage * kBBytes));
#pragma unroll
          for (int ks = 0; ks < kBlockK / 16; ++ks) {
            // +32 bytes per 16-element K step inside the 128-byte swizzle row (encoded >> 4).
            tc_mma_ss(d_tmem, a_desc + 2u * ks, b_desc + 2u * ks, idesc, (kc | ks) != 0 ? 1u : 0u);
          }
          tc_commit(&bars->b_empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        tc_commit(&bars->acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 0..3)
    const int row_in_tile = warp * 32 + lane;
    const long long row = static_cast<long long>(m0) + row_in_tile;
    const bool row_ok = row < M;
    const int clip = row_ok ? static_cast<int>(row / ep.T) : 0;
    const int t = row_ok ? static_cast<int>(row % ep.T) : 0;
    // RoPE factors of this thread's frame, kept in registers for all heads of q and k.  The table's two
    // 32-wide halves are identical by construction (frequencies repeated), so only the first is read.
    float rc[32], rs[32];
    if (n_first < 4 && row_ok) {
      const float4* c4 = reinterpret_cast<const float4*>(ep.cos + clip * ep.cos_bstride + static_cast<long long>(t) * 64);
      const float4* s4 = reinterpret_cast<const float4*>(ep.sin + clip * ep.cos_bstride + static_cast<long long>(t) * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 c = __ldg(c4 + i), sn = __ldg(s4 + i);
        rc[4 * i] = c.x; rc[4 * i + 1] = c.y; rc[4 * i + 2] = c.z; rc[4 * i + 3] = c.w;
        rs[4 * i] = sn.x; rs[4 * i + 1] = sn.y; rs[4 * i + 2] = sn.z; rs[4 * i + 3] = sn.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) { rc[i] = 1.f; rs[i] = 0.f; }
    }
    long long ring_row = -1;
    if (ep.ring_k != nullptr && row_ok) {
      const int pos = ep.pos_base + (ep.clip_pos != nullptr ? ep.clip_pos[clip] : 0) + t;
      // Only the newest ring_slots frames of a clip land in the ring.
      if (t >= ep.T - ep.ring_slots) ring_row = static_cast<long long>(clip) * 8 * ep.ring_slots + pos % ep.ring_slots;
    }
    for (int nt = 0; nt < n_tiles_per_cta; ++nt) {
      const int buf = nt & 1;
      const uint32_t use = static_cast<uint32_t>(nt >> 1);
      const int ntile = n_first + nt;
      const int seg = ntile >> 1;              // 0 = q, 1 = k, 2 = v
      mbar_wait(&bars->acc_full[buf], use & 1u, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(buf * kBlockN);
      uint16_t* lin = seg == 0 ? ep.q : (seg == 1 ? ep.k : ep.v);
      uint16_t* ring = seg == 1 ? ep.ring_k : (seg == 2 ? ep.ring_v : nullptr);
#pragma unroll 1
      for (int hh = 0; hh < 4; ++hh) {
        const int head = (ntile & 1) * 4 + hh;
        uint4* lin_dst = (lin != nullptr && row_ok) ? reinterpret_cast<uint4*>(lin + row * 512 + head * 64) : nullptr;
        uint4* ring_dst = (ring != nullptr && ring_row >= 0)
                              ? reinterpret_cast<uint4*>(ring + (ring_row + static_cast<long long>(head) * ep.ring_slots) * 64)
                              : nullptr;
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
          // 16 columns of the head's first half and the 16 columns 32 further on: a RoPE pair set.
          uint32_t lo[16], hi[16];
          tmem_ld16(t_row + hh * 64 + piece * 16, lo);
          tmem_ld16(t_row + hh * 64 + 32 + piece * 16, hi);
          tmem_ld_wait();
          uint32_t plo[8], phi[8];
          if (seg < 2) {
#pragma unroll
            for (int d = 0; d < 16; d += 2) {
              float o_lo[2], o_hi[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float a = __uint_as_float(lo[d + e]), b = __uint_as_float(hi[d + e]);
                const float c = rc[piece * 16 + d + e], sn = rs[piece * 16 + d + e];
                o_lo[e] = a * c - b * sn;
                o_hi[e] = b * c + a * sn;
              }
              plo[d / 2] = Pack16<__nv_bfloat16>::pack(o_lo[0], o_lo[1]);
              phi[d / 2] = Pack16<__nv_bfloat16>::pack(o_hi[0], o_hi[1]);
            }
          } else {
#pragma unroll
            for (int d = 0; d < 16; d += 2) {
              plo[d / 2] = Pack16<VT>::pack(__uint_as_float(lo[d]), __uint_as_float(lo[d + 1]));
              phi[d / 2] = Pack16<VT>::pack(__uint_as_float(hi[d]), __uint_as_float(hi[d + 1]));
            }
          }
          if (lin_dst != nullptr) {
            lin_dst[piece * 2] = make_uint4(plo[0], plo[1], plo[2], plo[3]);
            lin_dst[piece * 2 + 1] = make_uint4(plo[4], plo[5], plo[6], plo[7]);
            lin_dst[4 + piece * 2] = make_uint4(phi[0], phi[1], phi[2], phi[3]);
            lin_dst[4 + piece * 2 + 1] = make_uint4(phi[4], phi[5], phi[6], phi[7]);
          }
          if (ring_dst != nullptr) {
            ring_dst[piece * 2] = make_uint4(plo[0], plo[1], plo[2], plo[3]);
            ring_dst[piece * 2 + 1] = make_uint4(plo[4], plo[5], plo[6], plo[7]);
            ring_dst[4 + piece * 2] = make_uint4(phi[0], phi[1], phi[2], phi[3]);
            ring_dst[4 + piece * 2 + 1] = make_uint4(phi[4], phi[5], phi[6], phi[7]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
    }
  }

  // Teardown: every thread arrives here; the allocating warp releases tensor memory.
  tc_fence_before_sync();
  __syncthreads();
  if (ctl->abort) {
    // Give copies that may still be in flight time to land before shared memory is reused.
    __nanosleep(20000);
  }
  if (warp == 4) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int encode_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                          uint32_t box_cols) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

int launch_qkv_rope_gemm(const void* x, const void* w_qkv, const QkvEpilogueArgs& ep, int M, int value_is_fp16,
                         int* status, cudaStream_t st) {
  using namespace gemm;
  if (M <= 0) return M == 0 ? 0 : -1;
  if (ep.T <= 0 || ep.cos == nullptr || ep.sin == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_qkv)) & 15u) return -3;
  CUtensorMap tmap_x, tmap_w;
  int rc = encode_2d_bf16(&tmap_x, x, static_cast<uint64_t>(M), kHidden, kBlockM, kBlockK);
  if (rc != 0) return rc;
  rc = encode_2d_bf16(&tmap_w, w_qkv, 1536, kHidden, kBlockN, kBlockK);
  if (rc != 0) return rc;
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  // Few frame tiles (streaming decode): split the six 256-wide output tiles over CTAs too.
  const int n_split = m_tiles >= 148 ? 1 : (m_tiles >= 50 ? 3 : 6);
  const int per_cta = 6 / n_split;
  dim3 grid(m_tiles, n_split);
  auto kern = value_is_fp16 ? qkv_rope_gemm_kernel<__half> : qkv_rope_gemm_kernel<__nv_bfloat16>;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (rc != 0) return rc;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tmap_x, tmap_w, ep, M, per_cta, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
