// Banded causal attention for long clips (T > 256 frames) with a window of 130..257 frames (Mimi: 250), sm_100a.
// Same contract as the general prefill kernel (fm_prefill.cu): rotated q, k (BF16) and v (16-bit) in
// [B, T, 512], output [B, T, 512]; replaces the masked SDPA call of the reference
// (src/fast_mimi/model.py:1860-1868 with the band of src/fast_mimi/model.py:1672-1676) for long sequences.
//
// With such a window the 128 queries of tile t see keys of exactly three 128-key tiles: t-2 (far), t-1 (mid)
// and t (diagonal).  A persistent CTA walks RUNS of consecutive query tiles of one (clip, head), so the K and
// V tiles it needs are already in shared memory from the previous two steps: a ring of four K tiles and four
// V tiles (tile u in slot u % 4); per step it loads only Q_t, K_t and V_t (48 KB for 128 frames), each byte
// once.  A run's first step also loads its two halo tiles.
//
// The step's three 128 x 128 score tiles are three JOBS, as in the whole-clip kernel (fm_prefill_clip.cu):
// tensor memory is four 128-column slots, job g = 3 * step + kind runs in slot g % 4 with softmax team g % 4;
// S = Q K^T is turned in place into 16-bit P, which the tensor core reads from tensor memory for O = P V.
// All three jobs belong to the same 128 query rows: the teams exchange row maxima (and later row sums)
// through shared memory, use one common maximum, and the tensor core accumulates the three P V products
// into the diagonal job's slot, whose team normalises and stores the rows.  The window gives warp w of the
// far job 4-w visible 32-key groups and warp w of the diagonal job w+1, so the four SM sub-partitions carry
// the same load.  Tiles before the clip's first frame are not loaded; their jobs run empty.
// Warps 0-15: softmax teams.  Warp 16: Q/K loads + score products.  Warp 17: P V products.  Warp 18: V loads.
#include "fm_attn_tile.cuh"
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace longclip {
using attn_tile::kD;
using attn_tile::kTile;
constexpr int kTileBytes = kTile * kD * 2;          // 16 KB
constexpr int kSlabBytes = 32 * 128;                // 32 rows x 64 x 16 bit
constexpr int kSlots = 4;
constexpr int kRing = 4;                            // K tiles and V tiles kept: t-2, t-1, t and the next step's
constexpr int kSoftmaxWarps = 4 * kSlots;
constexpr int kIssueWarps = 3;
constexpr int kThreads = (kSoftmaxWarps + kIssueWarps) * 32;
constexpr int kTmemCols = 128 * kSlots;
constexpr uint32_t kPCol = 0, kOCol = 64;           // inside a slot: P over the consumed S, then O

struct Shared {
  uint64_t qk_full[2];     // Q and the new K tile(s) of the step in this Q buffer have landed
  uint64_t v_full[2];      // the new V tile(s) of the step have landed
  uint64_t qk_done[2];     // the step's score products have completed: its Q buffer and its far K tile are dead
  uint64_t pv_done[2];     // the step's P V products have completed: its far V tile and its P slots are dead
  uint64_t out_done;       // the four staged slabs have been read by their TMA stores
  uint64_t s_full[kSlots];
  uint64_t p_full[kSlots];
  uint64_t o_full[kSlots];
  uint64_t slot_free[kSlots];   // the team is done with the slot's tensor memory (tested for diagonal jobs)
  uint64_t xm_full[4];     // the three partial row maxima of a step are published (12 warps)
  uint64_t xl_full[4];     // the row sums of the far and mid jobs are published (8 warps)
  uint32_t tmem_base;
  CtaCtl ctl;
  float xm[4][kTile][3];   // by step % 4
  float xl[4][kTile][2];
};
constexpr int kSmemBytes = 1024 + 2 * kRing * kTileBytes + 2 * kTileBytes + 4 * kSlabBytes +
                           static_cast<int>((sizeof(Shared) + 127) & ~size_t(127));
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");

// The tiles a CTA visits: runs r = blockIdx.x, blockIdx.x + gridDim.x, ...; run r = (clip, head, segment) covers
// query tiles [t0, t1) of that (clip, head).  Every role of the kernel walks the same sequence with the
// same step counter n, which the barrier phases are derived from.
struct Walk {
  int n_runs, n_seg, seg_tiles, n_tiles;
  int run, t, t0, t1, n;
  __device__ __forceinline__ Walk(int n_runs_, int n_seg_, int seg_tiles_, int n_tiles_)
      : n_runs(n_runs_), n_seg(n_seg_), seg_tiles(seg_tiles_), n_tiles(n_tiles_), run(static_cast<int>(blockIdx.x)), n(0) {
    open();
  }
  __device__ __forceinline__ void open() {
    if (run < n_runs) {
      t0 = (run % n_seg) * seg_tiles;
      t1 = t0 + seg_tiles < n_tiles ? t0 + seg_tiles : n_tiles;
      t = t0;
    }
  }
  __device__ __forceinline__ bool valid() const { return run < n_runs; }
  __device__ __forceinline__ bool first() const { return t == t0; }
  __device__ __forceinline__ int clip() const { return (run / n_seg) >> 3; }
  __device__ __forceinline__ int head() const { return (run / n_seg) & 7; }
  __device__ __forceinline__ int first_tile_loaded() const { return t0 - 2 > 0 ? t0 - 2 : 0; }   // run's oldest halo tile
  __device__ __forceinline__ void next() {
    ++n;
    if (++t >= t1) {
      run += static_cast<int>(gridDim.x);
      open();
    }
  }
};
}  // namespace longclip

template <typename VT>
__global__ void __launch_bounds__(longclip::kThreads, 1)
band_attn_long_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_out,
                      int n_runs, int n_seg, int seg_tiles, int n_tiles, int T, int window, float scale_log2e,
                      int* status) {
  using namespace longclip;
  using namespace attn_tile;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_k = smem;                              // kRing tiles
  uint8_t* smem_v = smem_k + kRing * kTileBytes;       // kRing tiles
  uint8_t* smem_q = smem_v + kRing * kTileBytes;       // two tiles
  uint8_t* smem_stage = smem_q + 2 * kTileBytes;       // four slabs
  Shared* sh = reinterpret_cast<Shared*>(smem_stage + 4 * kSlabBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->qk_full[i], 1);
      mbar_init(&sh->v_full[i], 1);
      mbar_init(&sh->qk_done[i], 1);
      mbar_init(&sh->pv_done[i], 1);
    }
    mbar_init(&sh->out_done, 4);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&sh->s_full[i], 1);
      mbar_init(&sh->p_full[i], 4);
      mbar_init(&sh->o_full[i], 1);
      mbar_init(&sh->slot_free[i], 4);
      mbar_init(&sh->xm_full[i], 12);
      mbar_init(&sh->xl_full[i], 8);
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

  auto job_phase = [](int g) { return static_cast<uint32_t>(g >> 2) & 1u; };
  auto step_phase = [](int n) { return static_cast<uint32_t>(n >> 1) & 1u; };

  if (warp >= kSoftmaxWarps) {
    // All 32 lanes of an issuing warp walk its loop and one elected lane issues copies, MMAs and commits:
    // warp-uniform control flow keeps the descriptors in uniform registers and the sequences issue faster than
    // from a single lane under a lane test.
    const int role = warp - kSoftmaxWarps;
    const bool one = elect_one();
    constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kD, Pack16<VT>::kFmt, Pack16<VT>::kFmt, 0, 1);
    auto slot_addr = [&](int g) { return tmem_base + static_cast<uint32_t>((g & 3) * kTile); };
    if (role == 0) {
      // ---------------------------------------------------------- Q / K loads + score products
      if (one) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
      }
      auto load_qk = [&](const Walk& w) {
        if (!one) return;
        const int b = w.n & 1;
        const int u_lo = w.first() ? w.first_tile_loaded() : w.t;     // K tiles u_lo .. t arrive with this step
        mbar_arrive_expect_tx(&sh->qk_full[b], static_cast<uint32_t>((w.t - u_lo + 2) * kTileBytes));
        tma_load_3d(smem_q + b * kTileBytes, &tmap_q, &sh->qk_full[b], w.head() * kD, w.t * kTile, w.clip());
        for (int u = u_lo; u <= w.t; ++u)
          tma_load_3d(smem_k + (u & 3) * kTileBytes, &tmap_k, &sh->qk_full[b], w.head() * kD, u * kTile, w.clip());
      };
      Walk cur(n_runs, n_seg, seg_tiles, n_tiles), nxt(n_runs, n_seg, seg_tiles, n_tiles);
      if (cur.valid()) {
        load_qk(cur);
        nxt.next();
      }
      for (; cur.valid(); cur.next(), nxt.next()) {
        const int n = cur.n;
        if (nxt.valid() && !nxt.first()) {
          // Step n+1 of the same run reuses the Q buffer of step n-1 and the ring slot of that step's far
          // tile; both are dead once step n-1's scores exist.
          if (n >= 1) mbar_wait(&sh->qk_done[(n + 1) & 1], step_phase(n - 1), ctl, status, kErrWaitMma);
          load_qk(nxt);
        }
        mbar_wait(&sh->qk_full[n & 1], step_phase(n), ctl, status, kErrWaitTma);
        const uint64_t qd = umma_desc_sw128(smem_u32(smem_q + (n & 1) * kTileBytes));
        for (int kind = 0; kind < 3; ++kind) {
          const int g = 3 * n + kind;
          if (g >= 4) {
            // The slot's previous job must be out of it: a far / mid job when the P V products that read its P
            // have completed, a diagonal job when its team has read O.
            const int gp = g - 4;
            if (gp % 3 != 2) mbar_wait(&sh->pv_done[(gp / 3) & 1], step_phase(gp / 3), ctl, status, kErrWaitMma);
            else mbar_wait(&sh->slot_free[gp & 3], job_phase(gp), ctl, status, kErrWaitConsumer);
          }
          tc_fence_after_sync();
          const int u = cur.t - 2 + kind;              // key tile of this job
          if (u >= 0) {
            const uint64_t kd = umma_desc_sw128(smem_u32(smem_k + (u & 3) * kTileBytes));
#pragma unroll
            for (int ks = 0; ks < kD / 16; ++ks)
              if (one) tc_mma_ss(slot_addr(g), qd + 2u * ks, kd + 2u * ks, idesc_qk, ks != 0);
          }
          if (one) {
            tc_commit(&sh->s_full[g & 3]);
            if (kind == 2) tc_commit(&sh->qk_done[n & 1]);
          }
        }
        if (nxt.valid() && nxt.first()) {
          // A new run: its tiles go into ring slots that this step's tiles may still occupy.
          mbar_wait(&sh->qk_done[n & 1], step_phase(n), ctl, status, kErrWaitMma);
          load_qk(nxt);
        }
      }
    } else if (role == 1) {
      // ---------------------------------------------------------- P V products
      for (Walk w(n_runs, n_seg, seg_tiles, n_tiles); w.valid(); w.next()) {
        const int n = w.n;
        mbar_wait(&sh->v_full[n & 1], step_phase(n), ctl, status, kErrWaitTma);
        for (int kind = 0; kind < 3; ++kind)
          mbar_wait(&sh->p_full[(3 * n + kind) & 3], job_phase(3 * n + kind), ctl, status, kErrWaitConsumer);
        tc_fence_after_sync();
        bool accumulate = false;
        for (int kind = 0; kind < 3; ++kind) {
          const int u = w.t - 2 + kind;
          if (u < 0) continue;
          // O (+)= P V: A = P from tensor memory (8 columns per 16 keys), B = V (MN-major, 2 KB per 16 keys)
          const uint64_t v = umma_desc_sw128(smem_u32(smem_v + (u & 3) * kTileBytes));
#pragma unroll
          for (int ks = 0; ks < kTile / 16; ++ks)
            if (one)
              tc_mma_ts(slot_addr(3 * n + 2) + kOCol, slot_addr(3 * n + kind) + kPCol + 8u * ks,
                        v + static_cast<uint64_t>(ks) * 128u, idesc_pv, (accumulate || ks != 0) ? 1u : 0u);
          accumulate = true;
        }
        if (one) {
          tc_commit(&sh->o_full[(3 * n + 2) & 3]);
          tc_commit(&sh->o_full[(3 * n + 1) & 3]);   // nobody waits on these two; one completion per slot use
          tc_commit(&sh->o_full[(3 * n) & 3]);
          tc_commit(&sh->pv_done[n & 1]);
        }
      }
    } else if (role == 2) {
      // ---------------------------------------------------------- V loads
      if (one) tma_prefetch_desc(&tmap_v);
      for (Walk w(n_runs, n_seg, seg_tiles, n_tiles); w.valid(); w.next()) {
        const int n = w.n, b = n & 1;
        int u_lo = w.t;
        if (w.first()) {
          // new run: every ring slot may hold a tile of the previous step
          if (n >= 1) mbar_wait(&sh->pv_done[(n - 1) & 1], step_phase(n - 1), ctl, status, kErrWaitMma);
          u_lo = w.first_tile_loaded();
        } else if (w.t - 2 >= w.t0) {
          // the slot held tile t-4, last read by step n-2 of this run
          mbar_wait(&sh->pv_done[b], step_phase(n - 2), ctl, status, kErrWaitMma);
        }
        if (one) {
          mbar_arrive_expect_tx(&sh->v_full[b], static_cast<uint32_t>((w.t - u_lo + 1) * kTileBytes));
          for (int u = u_lo; u <= w.t; ++u)
            tma_load_3d(smem_v + (u & 3) * kTileBytes, &tmap_v, &sh->v_full[b], w.head() * kD, u * kTile, w.clip());
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax teams
    const int team = warp >> 2;               // == slot
    const int lg = warp & 3;                  // TMEM lane group
    const int r = lg * 32 + lane;             // row of the tile == TMEM lane
    const uint32_t slot = tmem_base + static_cast<uint32_t>(team * kTile) + (static_cast<uint32_t>(lg * 32) << 16);
    for (Walk w(n_runs, n_seg, seg_tiles, n_tiles); w.valid(); w.next()) {
      const int n = w.n, x = n & 3;
      const uint32_t xph = static_cast<uint32_t>(n >> 2) & 1u;     // this exchange buffer's use number
      const int kind = ((team - 3 * n) % 4 + 4) % 4;               // the job of this step that runs in this team's slot
      if (kind == 3) continue;                                     // none: the slot belongs to a neighbouring step
      const int g = 3 * n + kind;
      const uint32_t ph = job_phase(g);
      const int w_row0 = w.t * kTile + lg * 32;                    // first frame held by this warp
      const int i = w_row0 + lane;
      const GroupVis vis(i, w_row0, (w.t - 2 + kind) * kTile, window);

      mbar_wait(&sh->s_full[team], ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      float m_raw = tile_row_max(slot, vis);                       // -inf for a job with nothing visible
      sh->xm[x][r][kind] = m_raw;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->xm_full[x]);
      mbar_wait(&sh->xm_full[x], xph, ctl, status, kErrWaitConsumer);
      m_raw = fmaxf(fmaxf(sh->xm[x][r][0], sh->xm[x][r][1]), sh->xm[x][r][2]);
      const float m_use = (m_raw == -INFINITY) ? 0.f : m_raw * scale_log2e;
      float l_row = tile_row_probs<VT>(slot, slot + kPCol, vis, scale_log2e, m_use);
      if (kind != 2) sh->xl[x][r][kind] = l_row;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sh->p_full[team]);
        if (kind != 2) {
          mbar_arrive(&sh->xl_full[x]);
          mbar_arrive(&sh->slot_free[team]);   // keeps the barrier's phase in step with the slot's use count
        }
      }
      if (kind != 2) continue;                 // the diagonal job's team finishes the rows

      mbar_wait(&sh->o_full[team], ph, ctl, status, kErrWaitMma);
      tc_fence_after_sync();
      mbar_wait(&sh->xl_full[x], xph, ctl, status, kErrWaitConsumer);
      l_row += sh->xl[x][r][0] + sh->xl[x][r][1];
      // The previous step's stores out of the slabs must have read them.
      uint8_t* slab = smem_stage + lg * kSlabBytes;
      if (n >= 1) mbar_wait(&sh->out_done, static_cast<uint32_t>(n - 1) & 1u, ctl, status, kErrWaitConsumer);
      stage_output_row<VT>(slot + kOCol, slab, lane, 1.f / l_row);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sh->slot_free[team]);
        if (w_row0 < T) {                      // frames past T are clipped by the map
          tma_store_3d(&tmap_out, slab, w.head() * kD, w_row0, w.clip());
          bulk_commit_group();
          bulk_wait_group_read<0>();
        }
        mbar_arrive(&sh->out_done);
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

static int encode_long_map(CUtensorMap* map, const void* base, int B, int T, uint32_t box_rows) {
  // [B, T, 512] 16-bit viewed as (512 fastest, T, B); box = 64 columns x box_rows frames of one clip.
  const cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(T) * 512 * 2};
  const cuuint32_t box[3] = {64, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

int launch_band_attn_long(const void* q, const void* k, const void* v, void* out, int B, int T, int window, float scale,
                          int value_is_fp16, int* status, cudaStream_t st) {
  using namespace longclip;
  // three key tiles per query tile: the window must reach into tile t-2 and not beyond it
  if (T <= 2 * kTile || B <= 0 || window <= kTile + 1 || window > 2 * kTile + 1) return -1;
  CUtensorMap tq, tk, tv, tout;
  int rc = encode_long_map(&tq, q, B, T, kTile);
  if (rc == 0) rc = encode_long_map(&tk, k, B, T, kTile);
  if (rc == 0) rc = encode_long_map(&tv, v, B, T, kTile);     // element size is what matters: 16 bit
  if (rc == 0) rc = encode_long_map(&tout, out, B, T, 32);
  if (rc != 0) return rc;
  auto kern = value_is_fp16 ? band_attn_long_kernel<__half> : band_attn_long_kernel<__nv_bfloat16>;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (rc != 0) return rc;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 1;
  // Runs: whole (clip, head) sequences when there are enough of them to occupy the SMs, else segments of
  // each sequence (a segment re-reads the two K / V tiles in front of it).
  const int n_tiles = (T + kTile - 1) / kTile;
  const long long seqs = static_cast<long long>(B) * 8;
  int want_seg = static_cast<int>(sms / seqs);
  if (want_seg < 1) want_seg = 1;
  if (want_seg > n_tiles) want_seg = n_tiles;
  const int seg_tiles = (n_tiles + want_seg - 1) / want_seg;
  const int n_seg = (n_tiles + seg_tiles - 1) / seg_tiles;
  const long long n_runs_ll = seqs * n_seg;
  if (n_runs_ll > 0x7fffffffLL) return -1;
  const int n_runs = static_cast<int>(n_runs_ll);
  const int grid = n_runs < sms ? n_runs : sms;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tq, tk, tv, tout, n_runs, n_seg, seg_tiles, n_tiles, T, window,
                                          scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
