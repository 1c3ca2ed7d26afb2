// Banded causal attention for whole clips of 128 < T <= 256 frames (Mimi's 10 s clips: T = 250), sm_100a.
// Same contract as the general prefill kernel (fm_prefill.cu): rotated q, k (BF16) and v (16-bit) in
// [B, T, 512], output [B, T, 512]; replaces the masked SDPA call of the reference
// (src/fast_mimi/model.py:1860-1868 with the band of src/fast_mimi/model.py:1672-1676).
//
// A persistent CTA takes (clip, head) items; an item's Q, K, V for both 128-frame halves (96 KB) arrive
// in one TMA batch and the next item's batch is in flight meanwhile (two buffers).  The causal band of an
// item is three 128 x 128 score tiles, handled as three uniform JOBS:
//     kind 0: rows 0-127 x keys 0-127     kind 1: rows 128-255 x keys 0-127     kind 2: rows 128-255 x keys 128-255
// Tensor memory is four 128-column SLOTS; job g runs in slot g % 4 with softmax team g % 4 (four warps,
// one query row per thread).  In a slot, S = Q K^T (FP32, 128 columns) is turned IN PLACE into the 16-bit
// probabilities P (columns 0-63), which the tensor core reads straight from tensor memory as the A operand
// of O = P V; O (FP32) lands in columns 64-127 of the slot.  So there is no shared-memory round trip for P,
// and up to four jobs are in flight: while one team exponentiates, the tensor core works on other slots.
// Rows 128-255 need both of their tiles, but the two jobs do not wait for each other: each uses the maximum
// of its own tile, its P V product lands in its own slot, and the kind-2 team combines the two partial
// results at the end:  out = (a1 O1 + a2 O2) / (a1 l1 + a2 l2),  a_k = 2^(m_k - max(m1, m2)).  The causal
// diagonal leaves warp w of a kind-0 job 4-w visible 32-key groups (its frames are
// loaded in permuted order) and warp w of a kind-2 job w+1, which balances the four SM sub-partitions.
// Outputs are normalised, staged in the item's dead Q tiles and leave through TMA stores.
// Warps 0-15: softmax teams.  Warps 16-18: Q/K loads + score products, P V products, V loads (one thread each).
#include "fm_attn_tile.cuh"
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace clip {
using attn_tile::kTile;
using attn_tile::kD;
constexpr int kTileBytes = kTile * kD * 2;          // 16 KB
constexpr int kSlabBytes = 32 * 128;                // 32 rows x 64 x 16 bit
constexpr int kSlots = 4;
constexpr int kSoftmaxWarps = 4 * kSlots;
constexpr int kIssueWarps = 3;
constexpr int kThreads = (kSoftmaxWarps + kIssueWarps) * 32;
constexpr int kTmemCols = 128 * kSlots;
constexpr uint32_t kPCol = 0, kOCol = 64;           // inside a slot: P over the consumed S, then O

struct Shared {
  uint64_t qk_full[2];     // Q0 Q1 K0 K1 of the item in this buffer have landed (64 KB)
  uint64_t v_full[2];      // V0 V1 of the item in this buffer have landed (32 KB)
  uint64_t qk_done[2];     // the item's three score products have completed: its Q / K tiles are dead
  uint64_t pv_done[2];     // the item's three P V products have completed: its V tiles are dead
  uint64_t out_done_a;     // rows 0-127 of an item: the four staged slabs have been read by their TMA stores
  uint64_t out_done_b[2];  // rows 128-255 (staged in the item's V1 tile): likewise, per V buffer
  uint64_t s_full[kSlots];
  uint64_t p_full[kSlots];
  uint64_t o_full[kSlots];
  uint64_t slot_free[kSlots];   // the slot's O has been read (a kind-1 slot's by the kind-2 team of the item)
  uint64_t xl_full[4];     // row maximum and sum of the kind-1 job are published (4 warps)
  uint32_t tmem_base;
  CtaCtl ctl;
  float xs[4][kTile][2];   // scaled row maximum (-inf: nothing visible) and row sum of the kind-1 job, by item % 4
};
// Shared memory: two Q/K buffers (4 tiles each), two V buffers (2 tiles each), four 4 KB output slabs for
// rows 0-127 (rows 128-255 are staged in the item's V1 tile, which only their own P V product reads).
// Q / K tiles are released as soon as the item's scores exist, V tiles when its P V products are done, so
// the loads of item n+2 start long before item n has finished.
constexpr int kQkBytes = 4 * kTileBytes, kVBytes = 2 * kTileBytes, kStageBytes = 4 * kSlabBytes;
constexpr int kSmemBytes = 1024 + 2 * kQkBytes + 2 * kVBytes + kStageBytes + static_cast<int>((sizeof(Shared) + 127) & ~size_t(127));
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");
}  // namespace clip

template <typename VT>
__global__ void __launch_bounds__(clip::kThreads, 1)
band_attn_clip_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_q32,
                      const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ CUtensorMap tmap_out, int n_items, int T, int window,
                      float scale_log2e, int* status) {
  using namespace clip;
  using namespace attn_tile;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_v = smem + 2 * kQkBytes;
  uint8_t* smem_stage = smem_v + 2 * kVBytes;
  Shared* sh = reinterpret_cast<Shared*>(smem_stage + kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->qk_full[i], 1);
      mbar_init(&sh->v_full[i], 1);
      mbar_init(&sh->qk_done[i], 1);
      mbar_init(&sh->pv_done[i], 1);
    }
    mbar_init(&sh->out_done_a, 4);
    mbar_init(&sh->out_done_b[0], 4);
    mbar_init(&sh->out_done_b[1], 4);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&sh->s_full[i], 1);
      mbar_init(&sh->p_full[i], 4);
      mbar_init(&sh->o_full[i], 1);
      mbar_init(&sh->slot_free[i], 4);
      mbar_init(&sh->xl_full[i], 4);
    }
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
  const int n_jobs = 3 * n_local;

  if (warp >= kSoftmaxWarps) {
    // ------------------------------------------------------------ three single-purpose issuing warps,
    // each a plain in-order loop with blocking waits.  All 32 lanes walk the loop and one elected lane issues the
    // copies, MMAs and commits: with warp-uniform control flow the descriptors stay in uniform registers, and a
    // wait / few MMAs / commit sequence issues a third faster than from a single lane under a lane test.
    //   warp 16: Q/K loads + score products      warp 17: P V products      warp 18: V loads
    const int role = warp - kSoftmaxWarps;
    const bool one = elect_one();
    constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kD, Pack16<VT>::kFmt, Pack16<VT>::kFmt, 0, 1);
    auto slot_addr = [&](int g) { return tmem_base + static_cast<uint32_t>((g & 3) * kTile); };
    auto job_phase = [](int g) { return static_cast<uint32_t>(g >> 2) & 1u; };
    auto item_phase = [](int n) { return static_cast<uint32_t>(n >> 1) & 1u; };
    // O (+)= P V for one job: A = P from tensor memory (8 columns per 16 keys), B = V (MN-major, 2 KB per 16 keys).
    auto issue_pv = [&](int g_p, int g_o, const uint8_t* v_tile, bool accumulate) {
      const uint64_t v = umma_desc_sw128(smem_u32(v_tile));
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks)
        if (one) tc_mma_ts(slot_addr(g_o) + kOCol, slot_addr(g_p) + kPCol + 8u * ks, v + static_cast<uint64_t>(ks) * 128u, idesc_pv,
                  (accumulate || ks != 0) ? 1u : 0u);
    };
    if (role == 0) {
      if (one) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_q32);
        tma_prefetch_desc(&tmap_k);
      }
      auto load_qk = [&](int n) {
        if (!one) return;
        const int item = blockIdx.x + n * gridDim.x;
        const int c = item >> 3, h = item & 7, b = n & 1;
        uint8_t* base = smem + b * kQkBytes;
        mbar_arrive_expect_tx(&sh->qk_full[b], kQkBytes);
        // Q0 in four 32-frame boxes, block j of the tile <- frames 96-32j .. 127-32j.
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_load_3d(base + j * kSlabBytes, &tmap_q32, &sh->qk_full[b], h * kD, (3 - j) * 32, c);
        tma_load_3d(base + 1 * kTileBytes, &tmap_q, &sh->qk_full[b], h * kD, kTile, c);
        tma_load_3d(base + 2 * kTileBytes, &tmap_k, &sh->qk_full[b], h * kD, 0, c);
        tma_load_3d(base + 3 * kTileBytes, &tmap_k, &sh->qk_full[b], h * kD, kTile, c);
      };
      if (n_local > 0) load_qk(0);
      for (int n = 0; n < n_local; ++n) {
        if (n + 1 < n_local) {
          // The other Q/K buffer held item n-1; its tiles are dead once that item's scores exist.
          if (n >= 1) mbar_wait(&sh->qk_done[(n + 1) & 1], item_phase(n - 1), ctl, status, kErrWaitMma);
          load_qk(n + 1);
        }
        mbar_wait(&sh->qk_full[n & 1], item_phase(n), ctl, status, kErrWaitTma);
        const uint8_t* base = smem + (n & 1) * kQkBytes;
        for (int kind = 0; kind < 3; ++kind) {
          const int g = 3 * n + kind;
          // The slot's previous job must be out of it: its O has been read.
          if (g >= 4) mbar_wait(&sh->slot_free[g & 3], job_phase(g - 4), ctl, status, kErrWaitConsumer);
          tc_fence_after_sync();
          const uint64_t qd = umma_desc_sw128(smem_u32(base + (kind == 0 ? 0 : 1) * kTileBytes));
          const uint64_t kd = umma_desc_sw128(smem_u32(base + (kind == 2 ? 3 : 2) * kTileBytes));
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks)
            if (one) tc_mma_ss(slot_addr(g), qd + 2u * ks, kd + 2u * ks, idesc_qk, ks != 0);
          if (one) {
            tc_commit(&sh->s_full[g & 3]);
            if (kind == 2) tc_commit(&sh->qk_done[n & 1]);
          }
        }
      }
    } else if (role == 1) {
      // every job's O = P V goes into its own slot, in job order
      for (int g = 0; g < n_jobs; ++g) {
        const int n = g / 3, kind = g % 3;
        if (kind == 0) mbar_wait(&sh->v_full[n & 1], item_phase(n), ctl, status, kErrWaitTma);
        mbar_wait(&sh->p_full[g & 3], job_phase(g), ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        issue_pv(g, g, smem_v + (n & 1) * kVBytes + (kind == 2 ? kTileBytes : 0), false);
        if (one) {
          tc_commit(&sh->o_full[g & 3]);
          if (kind == 2) tc_commit(&sh->pv_done[n & 1]);
        }
      }
    } else if (role == 2) {
      if (one) tma_prefetch_desc(&tmap_v);
      for (int n = 0; n < n_local; ++n) {
        const int b = n & 1;
        if (n >= 2) {
          // The buffer held item n-2: its P V products and the output staged in its V1 tile are done.
          mbar_wait(&sh->pv_done[b], item_phase(n - 2), ctl, status, kErrWaitMma);
          mbar_wait(&sh->out_done_b[b], item_phase(n - 2), ctl, status, kErrWaitConsumer);
        }
        const int item = blockIdx.x + n * gridDim.x;
        const int c = item >> 3, h = item & 7;
        uint8_t* base = smem_v + b * kVBytes;
        if (one) {
          mbar_arrive_expect_tx(&sh->v_full[b], kVBytes);
          tma_load_3d(base, &tmap_v, &sh->v_full[b], h * kD, 0, c);
          tma_load_3d(base + kTileBytes, &tmap_v, &sh->v_full[b], h * kD, kTile, c);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax teams
    const int team = warp >> 2;               // == slot
    const int lg = warp & 3;                  // TMEM lane group
    const int r = lg * 32 + lane;             // row of the tile == TMEM lane
    const uint32_t slot = tmem_base + static_cast<uint32_t>(team * kTile) + (static_cast<uint32_t>(lg * 32) << 16);
    for (int g = team; g < n_jobs; g += kSlots) {
      const int n = g / 3, kind = g % 3, x = n & 3;
      const uint32_t ph = static_cast<uint32_t>(g >> 2) & 1u;      // this slot's use number
      const uint32_t xph = static_cast<uint32_t>(n >> 2) & 1u;     // this exchange buffer's use number
      const int item = blockIdx.x + n * gridDim.x;
      const int c = item >> 3, h = item & 7;
      const int w_row0 = kind == 0 ? (3 - lg) * 32 : kTile + lg * 32;   // first frame held by this warp
      const int i = w_row0 + lane;
      const GroupVis vis(i, w_row0, kind == 2 ? kTile : 0, window);

      mbar_wait(&sh->s_full[team], ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      static_assert(kPCol == 0, "P is written over the scores from the slot's first column");
      float m_off;                             // the offset the probabilities were taken against (-inf: nothing visible)
      float l_row = tile_row_softmax_online<VT>(slot, vis, scale_log2e, m_off);
      if (kind == 1) {
        sh->xs[x][r][0] = m_off;
        sh->xs[x][r][1] = l_row;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sh->p_full[team]);
        if (kind == 1) mbar_arrive(&sh->xl_full[x]);
      }
      if (kind == 1) continue;                 // its O stays in the slot until the kind-2 team has combined it

      mbar_wait(&sh->o_full[team], ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      // Weights of the two partial results of rows 128-255 (kind 0: a single one).  The P V product of the
      // kind-1 job was issued before this job's, so it has completed as well.
      float c_own = 1.f / l_row, c_other = 0.f;
      const uint32_t other = tmem_base + static_cast<uint32_t>(((g - 1) & 3) * kTile) + (static_cast<uint32_t>(lg * 32) << 16);
      if (kind == 2) {
        mbar_wait(&sh->xl_full[x], xph, ctl, status, kErrWaitConsumer);
        const float m1 = sh->xs[x][r][0], l1 = sh->xs[x][r][1];
        const float m = fmaxf(m_off, m1);      // m_off is finite: a row of the diagonal tile sees itself
        const float a2 = ex2_approx(m_off - m);
        const float a1 = (m1 == -INFINITY) ? 0.f : ex2_approx(m1 - m);
        const float inv = 1.f / (a1 * l1 + a2 * l_row);
        c_own = a2 * inv;
        c_other = a1 * inv;
      }
      // Rows 0-127 are staged in a slab of their own (the previous item's store out of it must have read
      // it); rows 128-255 in the item's V1 tile, whose only reader, P11 V1, has completed (o_full).
      uint8_t* slab = (kind == 0 ? smem_stage : smem_v + (n & 1) * kVBytes + kTileBytes) + lg * kSlabBytes;
      if (kind == 0 && n >= 1) mbar_wait(&sh->out_done_a, static_cast<uint32_t>(n - 1) & 1u, ctl, status, kErrWaitConsumer);
      if (kind == 2) stage_output_row2<VT>(slot + kOCol, other + kOCol, slab, lane, c_own, c_other);
      else stage_output_row<VT>(slot + kOCol, slab, lane, c_own);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sh->slot_free[team]);
        if (kind == 2) mbar_arrive(&sh->slot_free[(g - 1) & 3]);
        if (w_row0 < T) {                      // frames past T are clipped by the map
          tma_store_3d(&tmap_out, slab, h * kD, w_row0, c);
          bulk_commit_group();
          bulk_wait_group_read<0>();
        }
        mbar_arrive(kind == 0 ? &sh->out_done_a : &sh->out_done_b[n & 1]);
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
