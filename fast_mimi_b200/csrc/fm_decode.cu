// Single-frame streaming decode over a per-stream KV ring (HBM-bound) for sm_100a.
//
//   out[s, h, :] = softmax_j( scale * q[s,h,:] . K_ring[s,h,j,:] ) V_ring[s,h,j,:]   over the valid slots
//
// Replaces the cached one-frame attention of the reference: MimiKVCache.update's concat-and-crop
// (src/fast_mimi/model.py:450-471) followed by SDPA with one query (src/fast_mimi/model.py:1860-1868).
// The reference keeps the last window-1 rotated K/V rows and concatenates the new row; here the ring
// has `window` slots, the projection epilogue has already written the new row into slot pos % window,
// and softmax does not depend on slot order, so the visible set is identical.
//
// Work item = (stream, head): 2 x slots x 128 B of ring (K then V).  A persistent CTA streams items
// through a 3-stage shared-memory ring with untiled TMA bulk copies issued by one producer thread.
// Two consumer groups of four warps take alternate items, so two items are being reduced while a
// third is in flight; inside a group the slots are dealt round-robin to the warps: 16-byte vector reads, FP32 dot
// products, warp-shuffle reductions, and a four-way merge of (max, sum, output) through shared memory.
//
// While the rings have only just begun to fill (at most 32 valid slots, known on the host when all streams share one
// position) items are short and the staged pipeline is bound by its per-item hand-offs, not by bandwidth; those
// steps take ring_decode_short_kernel instead: one warp per item, 16-byte loads straight from global memory,
// scores kept in registers, no shared memory, with enough resident warps to cover the load latency.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace dec {
constexpr int kMaxSlots = 256;
constexpr int kStages = 3;
constexpr int kWarps = 4;            // warps per consumer group
constexpr int kGroups = 2;
constexpr int kThreads = (kGroups * kWarps + 1) * 32;
constexpr int kRowBytes = 128;

struct Ctl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  CtaCtl ctl;
  alignas(16) uint16_t qrow[kStages][64];   // the item's 64 query values, copied in with its ring slices
  float merge_m[kGroups][2][kWarps];
  float merge_l[kGroups][2][kWarps];
  float merge_o[kGroups][2][kWarps][64];
};
}  // namespace dec

namespace dec {
// One warp's share of an item: scores of its slots against the query, their maximum, and the exp-weighted sum
// of the V rows (unnormalised).  kGuard: skip blocks of four turns that lie wholly past the valid slots.
template <typename VT, bool kGuard>
__device__ __forceinline__ void reduce_item(const uint8_t* ks, const uint8_t* vs, const float (&qf)[8], int nv, int gw,
                                            int grp, int chunk, float& m_w, float& l_w, float (&acc)[8]) {
  // Slots are dealt to the group's four warps in turns of four (slot = 16 * it + 4 * gw + grp), so a ring
  // that is still filling keeps all four busy; the 16 turns run as four blocks of four, and a block that
  // lies wholly past the valid slots is skipped by the whole warp.
  float sc[16];
  m_w = -INFINITY;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    if (!kGuard || blk * 64 + gw * 4 < nv) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int it = blk * 4 + j;
        const int row = it * 16 + gw * 4 + grp;
        float part = 0.f;
        if (row < nv) {
          const uint4 raw = *reinterpret_cast<const uint4*>(ks + row * kRowBytes + chunk * 16);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = Pack16<__nv_bfloat16>::unpack(w[e]);
            part = fmaf(qf[2 * e], f.x, part);
            part = fmaf(qf[2 * e + 1], f.y, part);
          }
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        sc[it] = row < nv ? part : -INFINITY;
        m_w = fmaxf(m_w, sc[it]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[blk * 4 + j] = -INFINITY;
    }
  }
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 8));
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 16));
  const float m_use = (m_w == -INFINITY) ? 0.f : m_w;
  l_w = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    if (!kGuard || blk * 64 + gw * 4 < nv) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int it = blk * 4 + j;
        const int row = it * 16 + gw * 4 + grp;
        if (row < nv) {
          const float p = ex2_approx(sc[it] - m_use);
          l_w += p;
          const uint4 raw = *reinterpret_cast<const uint4*>(vs + row * kRowBytes + chunk * 16);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = Pack16<VT>::unpack(w[e]);
            acc[2 * e] = fmaf(p, f.x, acc[2 * e]);
            acc[2 * e + 1] = fmaf(p, f.y, acc[2 * e + 1]);
          }
        }
      }
    }
  }
}
}  // namespace dec

template <typename VT>
__global__ void __launch_bounds__(dec::kThreads, 1)
ring_decode_attn_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ ring_k,
                        const uint16_t* __restrict__ ring_v, float* __restrict__ out,
                        const int* __restrict__ stream_pos, int pos_base, int n_items, int ring_slots,
                        float scale_log2e, int* status) {
  using namespace dec;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const uint32_t tile_bytes = static_cast<uint32_t>(ring_slots) * kRowBytes;   // one K or V slice
  Ctl* c = reinterpret_cast<Ctl*>(smem);
  uint8_t* stage_base = smem + ((sizeof(Ctl) + 127) & ~size_t(127));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&c->full[i], 1);
      mbar_init(&c->empty[i], kWarps);
    }
    c->ctl.abort = 0;
    fence_mbar_init();
  }
  __syncthreads();
  CtaCtl* ctl = &c->ctl;

  // Slots 0..pos while the ring fills, all of them once it has wrapped.  A negative position (a caller
  // error that only a device-side stream_pos can still carry past the host checks) is recorded as
  // kErrBounds and the item reads slot 0 only, so no copy size or address is ever derived from it.
  auto valid_slots = [&](int item) {
    const int s = item >> 3;
    const int pos = pos_base + (stream_pos != nullptr ? stream_pos[s] : 0);
    if (pos < 0) {
      if (status != nullptr) atomicMax(status, static_cast<int>(kErrBounds));
      return 1;
    }
    return pos + 1 < ring_slots ? pos + 1 : ring_slots;
  };

  if (warp == kGroups * kWarps) {
    if (lane == 0) {
      int n = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
        const int st = n % kStages;
        const uint32_t use = static_cast<uint32_t>(n / kStages);
        mbar_wait(&c->empty[st], (use & 1u) ^ 1u, ctl, status, kErrWaitConsumer);
        const uint32_t bytes = static_cast<uint32_t>(valid_slots(item)) * kRowBytes;
        mbar_arrive_expect_tx(&c->full[st], 2 * bytes + 128);
        bulk_load_1d(&c->qrow[st][0], q + static_cast<size_t>(item) * 64, 128, &c->full[st]);
        const size_t src = static_cast<size_t>(item) * ring_slots * 64;
        bulk_load_1d(stage_base + (2 * st) * tile_bytes, ring_k + src, bytes, &c->full[st]);
        bulk_load_1d(stage_base + (2 * st + 1) * tile_bytes, ring_v + src, bytes, &c->full[st]);
      }
    }
  } else {
    const int chunk = lane & 7;    // which 8 of the 64 head dimensions this lane owns
    const int grp = lane >> 3;     // which of 4 consecutive slots
    const int cg = warp / kWarps;  // consumer group: takes items cg, cg + kGroups, ...
    const int gw = warp % kWarps;  // warp inside the group
    const int gt = threadIdx.x - cg * kWarps * 32;
    int n = cg;
    for (long long item = blockIdx.x + static_cast<long long>(cg) * gridDim.x; item < n_items;
         item += static_cast<long long>(kGroups) * gridDim.x, n += kGroups) {
      const int st = n % kStages;
      const uint32_t use = static_cast<uint32_t>(n / kStages);
      const int nv = valid_slots(static_cast<int>(item));
      const int s = static_cast<int>(item >> 3), h = static_cast<int>(item & 7);
      mbar_wait(&c->full[st], use & 1u, ctl, status, kErrWaitTma);
      const uint8_t* ks = stage_base + (2 * st) * tile_bytes;
      const uint8_t* vs = stage_base + (2 * st + 1) * tile_bytes;
      float qf[8];
      {
        const uint4 raw = *reinterpret_cast<const uint4*>(&c->qrow[st][chunk * 8]);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Pack16<__nv_bfloat16>::unpack(w[e]);
          qf[2 * e] = f.x * scale_log2e;
          qf[2 * e + 1] = f.y * scale_log2e;
        }
      }

      float m_w, l_w, acc[8];
      // A ring that is (nearly) full takes the loop without block guards: all 16 turns' loads can be in flight.
      if (nv > 3 * 64 + 3 * 4) reduce_item<VT, false>(ks, vs, qf, nv, gw, grp, chunk, m_w, l_w, acc);
      else reduce_item<VT, true>(ks, vs, qf, nv, gw, grp, chunk, m_w, l_w, acc);
      // Shared-memory reads of this stage are done: hand it back to the producer.
      __syncwarp();
      if (lane == 0) mbar_arrive(&c->empty[st]);

      l_w += __shfl_xor_sync(0xffffffffu, l_w, 8);
      l_w += __shfl_xor_sync(0xffffffffu, l_w, 16);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 8);
        acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
      }
      const int mb = (n / kGroups) & 1;
      if (grp == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) c->merge_o[cg][mb][gw][chunk * 8 + e] = acc[e];
        if (chunk == 0) {
          c->merge_m[cg][mb][gw] = m_w;
          c->merge_l[cg][mb][gw] = l_w;
        }
      }
      named_bar_sync(1 + cg, kWarps * 32);
      if (gt < 64) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, c->merge_m[cg][mb][w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float f = ex2_approx(c->merge_m[cg][mb][w] - mx);   // 0 for a warp that saw no slot
          num = fmaf(f, c->merge_o[cg][mb][w][gt], num);
          den = fmaf(f, c->merge_l[cg][mb][w], den);
        }
        out[static_cast<size_t>(s) * 512 + h * 64 + gt] = num / den;
      }
    }
  }
  __syncthreads();
  if (ctl->abort) __nanosleep(20000);
}

namespace dec {
constexpr int kShortMaxSlots = 32;      // valid slots up to which the one-warp-per-item kernel is used
constexpr int kShortWarps = 8;          // warps per block
}  // namespace dec

template <typename VT>
__global__ void __launch_bounds__(dec::kShortWarps * 32)
ring_decode_short_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ ring_k,
                         const uint16_t* __restrict__ ring_v, float* __restrict__ out, int nv, int n_items,
                         int ring_slots, float scale_log2e) {
  using namespace dec;
  const int lane = threadIdx.x & 31;
  const int chunk = lane & 7;    // which 8 of the 64 head dimensions this lane owns
  const int grp = lane >> 3;     // which of 4 consecutive slots
  const long long warp0 = static_cast<long long>(blockIdx.x) * kShortWarps + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * kShortWarps;
  constexpr int kIters = kShortMaxSlots / 4;
  for (long long item = warp0; item < n_items; item += stride) {
    const uint16_t* kb = ring_k + static_cast<size_t>(item) * ring_slots * 64 + chunk * 8;
    const uint16_t* vb = ring_v + static_cast<size_t>(item) * ring_slots * 64 + chunk * 8;
    float qf[8];
    {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q + static_cast<size_t>(item) * 64 + chunk * 8));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = Pack16<__nv_bfloat16>::unpack(w[e]);
        qf[2 * e] = f.x * scale_log2e;
        qf[2 * e + 1] = f.y * scale_log2e;
      }
    }
    float sc[kIters];
    float m_w = -INFINITY;
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      sc[it] = -INFINITY;
      if (it * 4 < nv) {               // the same for every lane
        const int row = it * 4 + grp;
        float part = 0.f;
        if (row < nv) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kb + static_cast<size_t>(row) * 64);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = Pack16<__nv_bfloat16>::unpack(w[e]);
            part = fmaf(qf[2 * e], f.x, part);
            part = fmaf(qf[2 * e + 1], f.y, part);
          }
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        if (row < nv) sc[it] = part;
        m_w = fmaxf(m_w, sc[it]);
      }
    }
    m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 8));
    m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 16));    // slot 0 is always valid: finite
    float l_w = 0.f;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int row = it * 4 + grp;
      if (it * 4 < nv && row < nv) {
        const float p = ex2_approx(sc[it] - m_w);
        l_w += p;
        const uint4 raw = *reinterpret_cast<const uint4*>(vb + static_cast<size_t>(row) * 64);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Pack16<VT>::unpack(w[e]);
          acc[2 * e] = fmaf(p, f.x, acc[2 * e]);
          acc[2 * e + 1] = fmaf(p, f.y, acc[2 * e + 1]);
        }
      }
    }
    l_w += __shfl_xor_sync(0xffffffffu, l_w, 8);
    l_w += __shfl_xor_sync(0xffffffffu, l_w, 16);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 8);
      acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
    }
    if (grp == 0) {
      const float inv = 1.f / l_w;
      float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(item) * 64 + chunk * 8);
      dst[0] = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
      dst[1] = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
    }
  }
}

int launch_ring_decode_attn(const void* q, const void* ring_k, const void* ring_v, float* out,
                            const int* stream_pos, int pos_base, int S, int ring_slots, float scale,
                            int value_is_fp16, int* status, cudaStream_t st) {
  using namespace dec;
  if (S <= 0) return S == 0 ? 0 : -1;
  if (ring_slots <= 0 || ring_slots > kMaxSlots || S > (1 << 27) || pos_base < 0) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(ring_k) | reinterpret_cast<uintptr_t>(ring_v)) & 15u)
    return -3;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = S * 8;
  if (stream_pos == nullptr && pos_base >= 0 && pos_base + 1 <= kShortMaxSlots && pos_base + 1 <= ring_slots) {
    // every ring holds slots 0..pos_base: short items, one warp each
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return -3;
    auto kern = value_is_fp16 ? ring_decode_short_kernel<__half> : ring_decode_short_kernel<__nv_bfloat16>;
    const long long want = (static_cast<long long>(n_items) + kShortWarps - 1) / kShortWarps;
    const long long cap = static_cast<long long>(sms > 0 ? sms : 1) * 8;
    kern<<<static_cast<int>(want < cap ? want : cap), kShortWarps * 32, 0, st>>>(
        static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(ring_k), static_cast<const uint16_t*>(ring_v), out,
        pos_base + 1, n_items, ring_slots, scale * 1.4426950408889634f);
    return static_cast<int>(cudaGetLastError());
  }
  const int smem_bytes = 128 + static_cast<int>((sizeof(Ctl) + 127) & ~size_t(127)) + kStages * 2 * ring_slots * kRowBytes;
  auto kern = value_is_fp16 ? ring_decode_attn_kernel<__half> : ring_decode_attn_kernel<__nv_bfloat16>;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes);
  if (rc != 0) return rc;
  const int grid = n_items < sms ? n_items : sms;
  kern<<<grid, kThreads, smem_bytes, st>>>(static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(ring_k),
                                          static_cast<const uint16_t*>(ring_v), out, stream_pos, pos_base,
                                          n_items, ring_slots, scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
