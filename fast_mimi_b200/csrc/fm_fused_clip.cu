// Projection + RoPE + banded causal attention in ONE kernel for clips of 128 < T <= 256 frames (Mimi's 10 s
// clips: T = 250), sm_100a.  x [B, T, 512] and W_qkv [1536, 512] in, attention output [B, T, 512] out: the rotated
// q, k and v never leave the SM.  Replaces, for such clips, the whole cache-free body of the reference's
// MimiAttention.forward before o_proj (src/fast_mimi/model.py:1897-1914 projections + _apply_rope, :1627-1688 band
// mask, :1860-1868 SDPA); the reference's own fused front half is src/fast_mimi/_packed_qkv.py:14-131,152-202.
//
// Two CTAs on neighbouring SMs (cluster of 2, tcgen05 cta_group::2) own one clip at a time: CTA r holds frames
// 128r .. 128r+127.  Each keeps its half of the clip's x resident in shared memory (128 KB, one TMA load per clip,
// the next clip's chunks replacing the current ones as the last head finishes with them) and walks the 8 heads:
//
//   projection   one pair MMA stream M = 256 frames x N = 192 (the head's q | k | v columns) x K = 512; each CTA
//                streams HALF of the head's W slice (96 rows, 12 KB stages), so a W byte crosses L2 -> SM once per
//                256 frames.  Accumulator: 192 TMEM columns per CTA.
//   epilogue     8 warps (two threads per frame row: RoPE pair sets 0-15 / 16-31, V dimensions 0-31 / 32-63):
//                RoPE in FP32, then  Q -> tensor memory (16-bit, 32 columns),
//                K -> this CTA's shared memory (128 keys x 64, K-major),  V -> TRANSPOSED into BOTH CTAs' shared
//                memory: dimensions 0-31 of every key to CTA 0, 32-63 to CTA 1 (V^T [32 d x 256 keys], K-major).
//   scores       one pair MMA M = 256, N = 256 keys, K = 64: A = Q from each CTA's tensor memory, B = K, each CTA
//                supplying its own 128 keys.  CTA r receives its 128 rows against all 256 keys; nothing is copied
//                between the CTAs.  (Rows 0-127 x keys 128-255 are computed and never read: causal.)
//   softmax      team A (4 warps) owns keys 0-127, team B keys 128-255 (only rows 128-255 need it).  Each uses its
//                own row maximum, writes the 16-bit probabilities in place over its scores, and the partial
//                results are combined at the end:  out = (a1 O1 + a2 O2) / (a1 l1 + a2 l2),  a = 2^(m - max).
//   P V          pair MMAs M = 256, N = 64, A = P from tensor memory, B = V^T: CTA s supplies output dimensions
//                32s .. 32s+31 for all keys, which is why V is stored split by dimension.
//   output       normalised in registers and written straight to global memory (128 contiguous bytes per frame-head).
//
// TMEM columns per CTA: [0,192) projection accumulator, [192,224) Q, [224,228) the teams' row maxima and sums,
// [256,512) scores (P and O overlay them).
// Warps: 0-7 epilogue, 8-11 team A, 12-15 team B, 16 W loads (+ TMEM allocation), 17 x loads, 18 projection MMAs
// (leader CTA), 19 attention MMAs (leader CTA).  Every barrier that gates a pair MMA lives in the leader and
// counts arrivals from both CTAs; completions are multicast to both.  No TMA multicast anywhere.
#include "fm_attn_tile.cuh"
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace fused {
using attn_tile::kD;
using attn_tile::kTile;
constexpr int kKChunks = 8;                       // 512 / 64
constexpr int kXChunkBytes = kTile * 64 * 2;      // 16 KB: 128 frames x 64 inputs
constexpr int kWStages = 4;
constexpr int kWRows = 96;                        // weight rows per CTA and head (half of q | k | v)
constexpr int kWBoxRows = 32;
constexpr int kWBoxBytes = kWBoxRows * 64 * 2;    // 4 KB
constexpr int kWStageBytes = kWRows * 64 * 2;     // 12 KB
constexpr int kKParkBytes = kTile * kD * 2;       // 16 KB
constexpr int kVtTileBytes = 32 * 64 * 2;         // 4 KB: 32 dimensions x 64 keys
constexpr int kVtBufBytes = 4 * kVtTileBytes;     // 16 KB: 256 keys
constexpr int kEpiWarps = 8;
constexpr int kTeamWarp0 = kEpiWarps;             // team A: warps 8-11, team B: warps 12-15
constexpr int kIssueWarp0 = kEpiWarps + 8;        // W loads, x loads, projection MMAs, attention MMAs
constexpr int kThreads = (kIssueWarp0 + 4) * 32;
constexpr int kTmemCols = 512;
constexpr uint32_t kAccCol = 0, kQCol = 192, kXCol = 224, kSCol = 256;   // kXCol: four columns for the teams' row maxima and sums
constexpr uint32_t kOOff = 64;                    // inside a team's 128 score columns: P at +0, O at +64

struct Shared {
  uint64_t x_full[kKChunks];    // leader: both CTAs' chunk kc of the clip has landed
  uint64_t x_empty[kKChunks];   // per CTA: the clip's last MMA over chunk kc has completed
  uint64_t w_full[kWStages];    // leader: both halves of a W stage have landed
  uint64_t w_empty[kWStages];   // per CTA: stage consumed
  uint64_t acc_full;            // per CTA: the head's projection is complete
  uint64_t acc_empty;           // leader: 16 epilogue warps have read the accumulator
  uint64_t park_full;           // leader: 16 epilogue warps have written Q, K and V^T of the head
  uint64_t qk_free;             // per CTA: the head's score MMAs have completed (Q and K may be overwritten)
  uint64_t v_free[2];           // per CTA: the head's P V MMAs have completed (this V^T buffer may be overwritten)
  uint64_t s_full;              // per CTA: scores are in tensor memory
  uint64_t p_full[2];           // leader: team A of both CTAs (8 warps) / team B of CTA 1 (4 warps) wrote P
  uint64_t o_full[2];           // per CTA: O_A / O_B complete
  uint64_t slot_free;           // leader: the 12 warps that read O (team A of CTA 0, both teams of CTA 1) are done with the score columns
  uint64_t xl_full;             // CTA 1: both teams (8 warps) published their row maxima and sums
  uint32_t tmem_base;
  uint32_t skip;
  CtaCtl ctl;
};
constexpr int kSharedBytes = static_cast<int>((sizeof(Shared) + 127) & ~size_t(127));
constexpr int kSmemBytes = 1024 + kKChunks * kXChunkBytes + kWStages * kWStageBytes + kKParkBytes + 2 * kVtBufBytes + kSharedBytes;
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");

// Row maximum of the visible raw scores (this thread's row of a 128 x 128 tile), two 32-column loads in flight.
__device__ __forceinline__ float tile_row_max_pipelined(uint32_t s_addr, const attn_tile::GroupVis& g) {
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  auto fold = [&](const uint32_t (&s)[32], int c0) {
    if (g.full(c0)) {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    } else {
#pragma unroll
      for (int cc = 0; cc < 32; ++cc)
        if (c0 + cc >= g.vis_lo && c0 + cc <= g.vis_hi) m[cc & 3] = fmaxf(m[cc & 3], __uint_as_float(s[cc]));
    }
  };
#pragma unroll 1
  for (int c0 = 0; c0 < kTile; c0 += 64) {
    const bool skip_a = g.skip(c0), skip_b = g.skip(c0 + 32);       // the same for every lane of the warp
    uint32_t a[32], b[32];
    if (!skip_a) tmem_ld32(s_addr + c0, a);
    if (!skip_b) tmem_ld32(s_addr + c0 + 32, b);
    if (!skip_a || !skip_b) tmem_ld_wait();
    if (!skip_a) fold(a, c0);
    if (!skip_b) fold(b, c0 + 32);
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// This thread's 64 output values from tensor memory, scaled and rounded to 32 packed words.
template <typename VT>
__device__ __forceinline__ void pack_output_row(uint32_t o_addr, float inv, uint32_t (&w)[32]) {
#pragma unroll
  for (int d0 = 0; d0 < kD; d0 += 32) {
    uint32_t o[32];
    tmem_ld32(o_addr + d0, o);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j)
      w[d0 / 2 + j] = Pack16<VT>::pack(__uint_as_float(o[2 * j]) * inv, __uint_as_float(o[2 * j + 1]) * inv);
  }
}
// Half of a row (32 output values) as the weighted sum of two partial outputs, 16 packed words.
template <typename VT>
__device__ __forceinline__ void pack_output_half2(uint32_t oa_addr, uint32_t ob_addr, float c_a, float c_b, uint32_t (&w)[16]) {
#pragma unroll
  for (int d0 = 0; d0 < 32; d0 += 16) {
    uint32_t oa[16], ob[16];
    tmem_ld16(oa_addr + d0, oa);
    tmem_ld16(ob_addr + d0, ob);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[d0 / 2 + j] = Pack16<VT>::pack(fmaf(__uint_as_float(oa[2 * j]), c_a, __uint_as_float(ob[2 * j]) * c_b),
                                       fmaf(__uint_as_float(oa[2 * j + 1]), c_a, __uint_as_float(ob[2 * j + 1]) * c_b));
  }
}
}  // namespace fused

template <typename VT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(fused::kThreads, 1)
attn_fused_clip_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                       const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, long long cos_bstride,
                       uint16_t* __restrict__ out, int n_clips, int T, int window, float scale_log2e,
                       uint32_t idesc_proj, int* status) {
  using namespace fused;
  using namespace attn_tile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_x = smem;                                        // 8 x [128 frames x 128 B]
  uint8_t* smem_w = smem_x + kKChunks * kXChunkBytes;            // kWStages x [96 rows x 128 B]
  uint8_t* smem_k = smem_w + kWStages * kWStageBytes;            // [128 keys x 128 B]
  uint8_t* smem_vt = smem_k + kKParkBytes;                       // 2 x 4 x [32 dims x 128 B (64 keys)]
  Shared* sh = reinterpret_cast<Shared*>(smem_vt + 2 * kVtBufBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int pair = static_cast<int>(blockIdx.x >> 1), n_pairs = static_cast<int>(gridDim.x >> 1);
  const int n_local = (n_clips - pair + n_pairs - 1) / n_pairs;   // clips pair, pair + n_pairs, ...
  const int n_heads_total = 8 * n_local;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kKChunks; ++i) {
      mbar_init(&sh->x_full[i], 1);
      mbar_init(&sh->x_empty[i], 1);
    }
    for (int i = 0; i < kWStages; ++i) {
      mbar_init(&sh->w_full[i], 1);
      mbar_init(&sh->w_empty[i], 1);
    }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->acc_empty, 2 * kEpiWarps);
    mbar_init(&sh->park_full, 2 * kEpiWarps);
    mbar_init(&sh->qk_free, 1);
    mbar_init(&sh->v_free[0], 1);
    mbar_init(&sh->v_free[1], 1);
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->p_full[0], 8);
    mbar_init(&sh->p_full[1], 4);
    mbar_init(&sh->o_full[0], 1);
    mbar_init(&sh->o_full[1], 1);
    mbar_init(&sh->slot_free, 12);
    mbar_init(&sh->xl_full, 8);
    sh->ctl.abort = 0;
    sh->skip = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 1u : 0u;
    fence_mbar_init();
  }
  if (warp == kIssueWarp0) {
    tmem_alloc_pair(&sh->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  CtaCtl* ctl = &sh->ctl;
  const bool skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&sh->skip), 0)) != 0;
  // Leader-side barriers as seen from either CTA.
  const uint32_t acc_empty_l = map_to_cta(smem_u32(&sh->acc_empty), 0);
  const uint32_t park_full_l = map_to_cta(smem_u32(&sh->park_full), 0);
  const uint32_t slot_free_l = map_to_cta(smem_u32(&sh->slot_free), 0);

  if (skip) {
    // a previous kernel already reported an error through this status word: do nothing
  } else if (warp == kIssueWarp0) {
    // ------------------------------------------------------------ W loads
    // In all four issuing warps the 32 lanes walk the loop together and one elected lane issues copies, MMAs and
    // commits: warp-uniform control flow keeps descriptors in uniform registers, and a wait / few MMAs / commit
    // sequence issues a third faster than from a single lane under a lane test.
    {
      const bool one = elect_one();
      if (one) tma_prefetch_desc(&tmap_w);
      int stage = 0;
      uint32_t phase = 0;
      for (int g = 0; g < n_heads_total; ++g) {
        const int h = g & 7;
        // This CTA's 96 of the head's 192 output columns, in accumulator order q (64) | k (64) | v (64):
        // CTA 0: q 0-31, q 32-63, k 0-31;  CTA 1: k 32-63, v 0-31, v 32-63.
        const int r0 = leader ? h * 64 : 512 + h * 64 + 32;
        const int r1 = leader ? h * 64 + 32 : 1024 + h * 64;
        const int r2 = leader ? 512 + h * 64 : 1024 + h * 64 + 32;
        for (int kc = 0; kc < kKChunks; ++kc) {
          mbar_wait(&sh->w_empty[stage], phase ^ 1u, ctl, status, kErrWaitConsumer);
          uint8_t* dst = smem_w + stage * kWStageBytes;
          if (one) {
            if (leader) mbar_arrive_expect_tx(&sh->w_full[stage], 2 * kWStageBytes);
            tma_load_2d_pair(dst, &tmap_w, &sh->w_full[stage], kc * 64, r0);
            tma_load_2d_pair(dst + kWBoxBytes, &tmap_w, &sh->w_full[stage], kc * 64, r1);
            tma_load_2d_pair(dst + 2 * kWBoxBytes, &tmap_w, &sh->w_full[stage], kc * 64, r2);
          }
          if (++stage == kWStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kIssueWarp0 + 1) {
    // ------------------------------------------------------------ x loads
    {
      const bool one = elect_one();
      if (one) tma_prefetch_desc(&tmap_x);
      for (int n = 0; n < n_local; ++n) {
        const int clip = pair + n * n_pairs;
        for (int kc = 0; kc < kKChunks; ++kc) {
          if (n > 0) mbar_wait(&sh->x_empty[kc], static_cast<uint32_t>(n - 1) & 1u, ctl, status, kErrWaitMma);
          if (one) {
            if (leader) mbar_arrive_expect_tx(&sh->x_full[kc], 2 * kXChunkBytes);
            tma_load_3d_pair(smem_x + kc * kXChunkBytes, &tmap_x, &sh->x_full[kc], kc * 64, static_cast<int>(rank) * kTile, clip);
          }
        }
      }
    }
  } else if (warp == kIssueWarp0 + 2) {
    // ------------------------------------------------------------ projection MMAs (leader CTA only)
    if (leader) {
      const bool one = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int chunk = 0;                 // running count of K chunks issued
      for (int g = 0; g < n_heads_total; ++g) {
        const int n = g >> 3, h = g & 7;
        if (g >= 1) mbar_wait(&sh->acc_empty, static_cast<uint32_t>(g - 1) & 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        for (int kc = 0; kc < kKChunks; ++kc, ++chunk) {
          // The tensor core runs MMAs in issue order.  At most two chunks (8 MMAs) of projection are queued, so
          // that the attention MMAs of the other issuing warp, which sit on the critical path, wait behind
          // little: chunk c is issued once chunk c - 2 has completed.
          if (chunk >= 2)
            mbar_wait(&sh->w_empty[(chunk - 2) % kWStages], static_cast<uint32_t>((chunk - 2) / kWStages) & 1u, ctl, status,
                      kErrWaitMma);
          if (h == 0) mbar_wait(&sh->x_full[kc], static_cast<uint32_t>(n) & 1u, ctl, status, kErrWaitTma);
          mbar_wait(&sh->w_full[stage], phase, ctl, status, kErrWaitTma);
          tc_fence_after_sync();
          const uint64_t a_desc = umma_desc_sw128(smem_u32(smem_x + kc * kXChunkBytes));
          const uint64_t b_desc = umma_desc_sw128(smem_u32(smem_w + stage * kWStageBytes));
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            if (one) tc_mma_ss_pair(tmem_base + kAccCol, a_desc + 2u * ks, b_desc + 2u * ks, idesc_proj, (kc | ks) != 0 ? 1u : 0u);
          if (one) {
            tc_commit_pair(&sh->w_empty[stage], 3);
            if (h == 7) tc_commit_pair(&sh->x_empty[kc], 3);      // the clip's last use of this x chunk
          }
          if (++stage == kWStages) { stage = 0; phase ^= 1u; }
        }
        if (one) tc_commit_pair(&sh->acc_full, 3);
      }
    }
  } else if (warp == kIssueWarp0 + 3) {
    // ------------------------------------------------------------ attention MMAs (leader CTA only)
    if (leader) {
      const bool one = elect_one();
      constexpr uint32_t idesc_s = umma_idesc_f16(2 * kTile, 2 * kTile, 1, 1, 0, 0);                        // bf16 q, k
      constexpr uint32_t idesc_pv = umma_idesc_f16(2 * kTile, kD, Pack16<VT>::kFmt, Pack16<VT>::kFmt, 0, 0);  // V^T is K-major
      const uint64_t k_desc = umma_desc_sw128(smem_u32(smem_k));
      for (int g = 0; g < n_heads_total; ++g) {
        const uint32_t ph = static_cast<uint32_t>(g) & 1u;
        mbar_wait_cluster(&sh->park_full, ph, ctl, status, kErrWaitConsumer);
        if (g >= 1) mbar_wait(&sh->slot_free, ph ^ 1u, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          if (one) tc_mma_ts_pair(tmem_base + kSCol, tmem_base + kQCol + 8u * ks, k_desc + 2u * ks, idesc_s, ks != 0 ? 1u : 0u);
        if (one) {
          tc_commit_pair(&sh->s_full, 3);
          tc_commit_pair(&sh->qk_free, 3);
        }
        const uint64_t v_desc = umma_desc_sw128(smem_u32(smem_vt + (g & 1) * kVtBufBytes));
#pragma unroll 1
        for (int team = 0; team < 2; ++team) {
          mbar_wait_cluster(&sh->p_full[team], ph, ctl, status, kErrWaitConsumer);
          tc_fence_after_sync();
          const uint32_t p_addr = tmem_base + kSCol + static_cast<uint32_t>(team * kTile);
#pragma unroll
          for (int ks = 0; ks < kTile / 16; ++ks) {
            // keys 128 team + 16 ks ..: tile (2 team + ks / 4) of V^T, 32 bytes per 16 keys inside the tile
            const uint64_t b = v_desc + static_cast<uint64_t>((2 * team + (ks >> 2)) * (kVtTileBytes >> 4)) + 2u * (ks & 3);
            if (one) tc_mma_ts_pair(p_addr + kOOff, p_addr + 8u * ks, b, idesc_pv, ks != 0 ? 1u : 0u);
          }
          if (one) tc_commit_pair(&sh->o_full[team], 3);
        }
        if (one) tc_commit_pair(&sh->v_free[g & 1], 3);
      }
    }
  } else if (warp < kEpiWarps) {
    // ------------------------------------------------------------ epilogue: two threads per frame row; `half`
    // selects RoPE pair set 16 half .. 16 half + 15 (dimensions d and d + 32) of q and k, and dimensions
    // 32 half .. 32 half + 31 of v (which are the rows of CTA `half`'s V^T).
    const int lg = warp & 3, half = warp >> 2;
    const int row = lg * 32 + lane;
    const int frame = static_cast<int>(rank) * kTile + row;         // also the key index of this row's K and V
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lg * 32) << 16);
    float rc[16], rs[16];
    auto load_tables = [&](int clip) {
      if (frame < T) {
        const float4* c4 = reinterpret_cast<const float4*>(cos_tab + clip * cos_bstride + static_cast<long long>(frame) * 64 + half * 16);
        const float4* s4 = reinterpret_cast<const float4*>(sin_tab + clip * cos_bstride + static_cast<long long>(frame) * 64 + half * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 c = __ldg(c4 + j), sn = __ldg(s4 + j);
          rc[4 * j] = c.x; rc[4 * j + 1] = c.y; rc[4 * j + 2] = c.z; rc[4 * j + 3] = c.w;
          rs[4 * j] = sn.x; rs[4 * j + 1] = sn.y; rs[4 * j + 2] = sn.z; rs[4 * j + 3] = sn.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) { rc[j] = 1.f; rs[j] = 0.f; }
      }
    };
    if (cos_bstride == 0) load_tables(0);
    // V^T destinations: dimension d of this key goes to CTA d / 32, row d % 32 of tile key / 64, at byte
    // ((key % 64) / 8 ^ (d % 8)) * 16 + (key % 8) * 2 of the 128-byte row (the 128-byte swizzle).
    const uint32_t vt_cta = map_to_cta(smem_u32(smem_vt), static_cast<uint32_t>(half));
    const uint32_t vt_key = static_cast<uint32_t>((frame >> 6) * kVtTileBytes + (frame & 7) * 2);
    const uint32_t vt_chunk = static_cast<uint32_t>((frame & 63) >> 3);
    for (int g = 0; g < n_heads_total; ++g) {
      const uint32_t ph = static_cast<uint32_t>(g) & 1u;
      if ((g & 7) == 0 && cos_bstride != 0) load_tables(pair + (g >> 3) * n_pairs);
      mbar_wait(&sh->acc_full, ph, ctl, status, kErrWaitMma);
      // Q and K of the previous head must have been consumed by its score MMAs.
      if (g >= 1) mbar_wait(&sh->qk_free, ph ^ 1u, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
#pragma unroll
      for (int seg = 0; seg < 2; ++seg) {          // 0 = q -> tensor memory, 1 = k -> shared memory
        {
          const int piece = half;
          // 16 columns of the first half of the head and the 16 columns 32 further on: a RoPE pair set
          uint32_t lo[16], hi[16];
          tmem_ld16(t_row + kAccCol + seg * 64 + piece * 16, lo);
          tmem_ld16(t_row + kAccCol + seg * 64 + 32 + piece * 16, hi);
          tmem_ld_wait();
          uint32_t plo[8], phi[8];
#pragma unroll
          for (int d = 0; d < 16; d += 2) {
            float o_lo[2], o_hi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float a = __uint_as_float(lo[d + e]), b = __uint_as_float(hi[d + e]);
              const float c = rc[d + e], sn = rs[d + e];
              o_lo[e] = a * c - b * sn;
              o_hi[e] = b * c + a * sn;
            }
            plo[d / 2] = Pack16<__nv_bfloat16>::pack(o_lo[0], o_lo[1]);
            phi[d / 2] = Pack16<__nv_bfloat16>::pack(o_hi[0], o_hi[1]);
          }
          if (seg == 0) {
            tmem_st8(t_row + kQCol + piece * 8, plo);             // dimensions 16 piece .. : 2 per column
            tmem_st8(t_row + kQCol + 16 + piece * 8, phi);        // dimensions 32 + 16 piece ..
          } else {
            *reinterpret_cast<uint4*>(smem_k + sw128_offset(row, piece * 2)) = make_uint4(plo[0], plo[1], plo[2], plo[3]);
            *reinterpret_cast<uint4*>(smem_k + sw128_offset(row, piece * 2 + 1)) = make_uint4(plo[4], plo[5], plo[6], plo[7]);
            *reinterpret_cast<uint4*>(smem_k + sw128_offset(row, 4 + piece * 2)) = make_uint4(phi[0], phi[1], phi[2], phi[3]);
            *reinterpret_cast<uint4*>(smem_k + sw128_offset(row, 4 + piece * 2 + 1)) = make_uint4(phi[4], phi[5], phi[6], phi[7]);
          }
        }
      }
      // V^T buffer g % 2 was last read by the P V products of head g - 2.
      if (g >= 2) mbar_wait(&sh->v_free[g & 1], (static_cast<uint32_t>(g >> 1) & 1u) ^ 1u, ctl, status, kErrWaitMma);
      const uint32_t vt_buf = static_cast<uint32_t>((g & 1) * kVtBufBytes) + vt_key;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        const int q4 = 2 * half + q2;
        uint32_t vv[16];
        tmem_ld16(t_row + kAccCol + 128 + q4 * 16, vv);
        tmem_ld_wait();
        if (q2 == 1) {
          // last read of the accumulator: hand it back before the stores (the loads have completed, so the
          // arrival needs no release ordering)
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty_l);
        }
        const uint32_t dst = vt_cta + vt_buf;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int dr = q2 * 16 + j;                              // row of the V^T tile
          const uint32_t v16 = Pack16<VT>::pack(__uint_as_float(vv[j]), 0.f) & 0xFFFFu;
          st_shared_cluster_u16(dst + static_cast<uint32_t>(dr * 128) + ((vt_chunk ^ static_cast<uint32_t>(dr & 7)) << 4),
                                static_cast<uint16_t>(v16));
        }
      }
      tmem_st_wait();
      fence_proxy_async_all();      // K and V^T stores (this CTA's and the partner's shared memory) -> tensor core
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(park_full_l);
    }
  } else if (!(warp >= kTeamWarp0 + 4 && leader)) {
    // ------------------------------------------------------------ softmax teams (team B only where rows see keys >= 128)
    const int team = (warp - kTeamWarp0) >> 2;  // 0: keys 0-127, 1: keys 128-255
    const int lg = warp & 3;
    const int w_row0 = static_cast<int>(rank) * kTile + lg * 32;
    const int i = w_row0 + lane;                // this thread's frame
    const uint32_t lane_sel = static_cast<uint32_t>(lg * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_sel + kSCol + static_cast<uint32_t>(team * kTile);
    const uint32_t sa_addr = tmem_base + lane_sel + kSCol;      // team A's columns (CTA 1's team B reads O_A there)
    const uint32_t p_full_l = map_to_cta(smem_u32(&sh->p_full[team]), 0);
    const GroupVis vis(i, w_row0, team * kTile, window);
    // Rows 128-255 (CTA 1) have two partial results, team A's over keys 0-127 and team B's over keys 128-255.  The
    // teams exchange their row maxima and sums through four spare tensor-memory columns and each finishes HALF of
    // every row (team A output dimensions 0-31, team B 32-63), so the combine and the global stores, which sit
    // between one head's P V product and the next head's scores, are shared by eight warps instead of four.
    const bool two_parts = !leader;
    const uint32_t x_addr = tmem_base + lane_sel + kXCol;
    for (int g = 0; g < n_heads_total; ++g) {
      const uint32_t ph = static_cast<uint32_t>(g) & 1u;
      mbar_wait(&sh->s_full, ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      float m_off;                    // the offset the probabilities were taken against (-inf: nothing visible)
      const float l_row = tile_row_softmax_online<VT>(s_addr, vis, scale_log2e, m_off);
      if (two_parts) {
        // offset and row sum of this team's part
        tmem_st1(x_addr + 2u * team, __float_as_uint(m_off));
        tmem_st1(x_addr + 2u * team + 1u, __float_as_uint(l_row));
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        // P (and the exchange columns) live in tensor memory and their stores have completed (tcgen05.wait::st), so
        // the arrivals order nothing; the release form would also wait for this thread's output stores in flight.
        mbar_arrive_cluster_relaxed(p_full_l);
        if (two_parts) mbar_arrive(&sh->xl_full);
      }

      // O_B was committed after O_A by the same thread, so in CTA 1 the wait for O_B covers both.
      mbar_wait(&sh->o_full[two_parts ? 1 : 0], ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      const int clip = pair + (g >> 3) * n_pairs, h = g & 7;
      uint16_t* dst = i < T ? out + (static_cast<long long>(clip) * T + i) * 512 + h * kD : nullptr;
      if (two_parts) {
        mbar_wait(&sh->xl_full, ph, ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        uint32_t x4[4];
        tmem_ld4(x_addr, x4);
        tmem_ld_wait();
        const float m_a = __uint_as_float(x4[0]), l_a = __uint_as_float(x4[1]);
        const float m_b = __uint_as_float(x4[2]), l_b = __uint_as_float(x4[3]);      // finite: a row sees itself
        const float m = fmaxf(m_a, m_b);
        const float c_b = ex2_approx(m_b - m);
        const float c_a = (m_a == -INFINITY) ? 0.f : ex2_approx(m_a - m);
        const float inv = 1.f / (c_a * l_a + c_b * l_b);
        uint32_t packed[16];
        pack_output_half2<VT>(sa_addr + kOOff + 32u * team, sa_addr + kTile + kOOff + 32u * team, c_a * inv, c_b * inv, packed);
        // The score columns are free as soon as O is in registers: the next head's scores do not wait for the
        // global stores.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(slot_free_l);
        if (dst != nullptr) {
#pragma unroll
          for (int c = 0; c < 2; ++c) st_global_v8(dst + 32 * team + 16 * c, &packed[8 * c]);
        }
      } else {
        uint32_t packed[32];
        pack_output_row<VT>(s_addr + kOOff, 1.f / l_row, packed);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(slot_free_l);
        if (dst != nullptr) {
#pragma unroll
          for (int c = 0; c < 4; ++c) st_global_v8(dst + 16 * c, &packed[8 * c]);
        }
      }
    }
  }

  // Teardown: neither CTA may leave (or release TMEM) while its partner can still signal it or store into it.
  tc_fence_before_sync();
  __syncthreads();
  if (ctl->abort) __nanosleep(20000);
  cluster_sync_all();
  if (warp == kIssueWarp0) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

int launch_attn_fused_clip(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                           void* out, int B, int T, int window, float scale, int dtype_flags, int* status,
                           cudaStream_t st) {
  using namespace fused;
  if (T <= kTile || T > 2 * kTile || B <= 0 || window <= 0 || cos == nullptr || sin == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_qkv) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin)) & 15u)
    return -3;
  CUtensorMap tmap_x, tmap_w;
  {
    // x [B, T, 512] viewed as (512 fastest, T, B): frames past the clip read as zero
    const cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(T) * 512 * 2};
    const cuuint32_t box[3] = {64, kTile, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const int rc = encode_tiled(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(x), dims, strides, box, estr,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  {
    const cuuint64_t dims[2] = {512, 1536};
    const cuuint64_t strides[1] = {512 * 2};
    const cuuint32_t box[2] = {64, kWBoxRows};
    const cuuint32_t estr[2] = {1, 1};
    const int rc = encode_tiled(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w_qkv), dims, strides, box, estr,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int max_pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int n_pairs = B < max_pairs ? B : max_pairs;
  // dtype_flags bit 0: v, P and the output are FP16 (else BF16); bit 1: x and w_qkv hold FP16 (else BF16).
  const int in_fmt = (dtype_flags & 2) ? 0 : 1;
  const uint32_t idesc_proj = umma_idesc_f16(2 * kTile, 192, in_fmt, in_fmt, 0, 0);
  auto kern = (dtype_flags & 1) ? attn_fused_clip_kernel<__half> : attn_fused_clip_kernel<__nv_bfloat16>;
  const int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (rc != 0) return rc;
  kern<<<2 * n_pairs, kThreads, kSmemBytes, st>>>(tmap_x, tmap_w, cos, sin, cos_bstride, static_cast<uint16_t*>(out), B, T,
                                                 window, scale * 1.4426950408889634f, idesc_proj, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
