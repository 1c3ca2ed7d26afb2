// KV-ring bookkeeping kernels for multi-frame cached calls (sm_100a, plain vector copies).
//
// The reference's cache keeps the last window-1 rotated K / V rows per layer, returns their concatenation with
// the call's new rows for this call's attention, then crops (MimiKVCache.update, src/fast_mimi/model.py:435-471).
// Here the persistent state is a ring [streams, 8 heads, slots, 64] whose slot p % slots holds the frame at
// absolute position p.  A call with T > 1 new frames at position `past` needs
//   ring_linearize:  k_lin[s, j, :] for j < delta  = ring row of position past - delta + j   (delta = min(past, W-1))
//                    k_lin[s, delta + t, :]        = the call's new row t                      (same for v)
//   ring_append:     the newest min(T, slots) new rows go to their slots (position past + t).
// Linearising BEFORE appending matters: a long chunk overwrites slots that its own first rows still attend to.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

// One thread per 16-byte piece (8 of the 64 values of one head of one frame); K and V in the same pass.
__global__ void __launch_bounds__(256)
ring_linearize_kernel(const uint4* __restrict__ ring_k, const uint4* __restrict__ ring_v, const uint4* __restrict__ k_new,
                      const uint4* __restrict__ v_new, uint4* __restrict__ k_lin, uint4* __restrict__ v_lin, int S, int T,
                      int delta, int past, int slots) {
  const int Tk = delta + T;
  const long long total = static_cast<long long>(S) * Tk * 64;      // 64 pieces per frame (8 heads x 8)
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int piece = static_cast<int>(i & 63);
    const long long frame = i >> 6;
    const int j = static_cast<int>(frame % Tk);
    const long long s = frame / Tk;
    uint4 kv, vv;
    if (j < delta) {
      const int slot = (past - delta + j) % slots;
      const long long src = ((s * 8 + (piece >> 3)) * slots + slot) * 8 + (piece & 7);
      kv = ring_k[src];
      vv = ring_v[src];
    } else {
      const long long src = (s * T + (j - delta)) * 64 + piece;
      kv = k_new[src];
      vv = v_new[src];
    }
    k_lin[i] = kv;
    v_lin[i] = vv;
  }
}

__global__ void __launch_bounds__(256)
ring_append_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new, uint4* __restrict__ ring_k,
                   uint4* __restrict__ ring_v, int S, int T, int t_first, int past, int slots) {
  const int n_t = T - t_first;                                      // rows t_first .. T-1 survive in the ring
  const long long total = static_cast<long long>(S) * n_t * 64;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int piece = static_cast<int>(i & 63);
    const long long frame = i >> 6;
    const int t = t_first + static_cast<int>(frame % n_t);
    const long long s = frame / n_t;
    const int slot = (past + t) % slots;
    const long long src = (s * T + t) * 64 + piece;
    const long long dst = ((s * 8 + (piece >> 3)) * slots + slot) * 8 + (piece & 7);
    ring_k[dst] = k_new[src];
    ring_v[dst] = v_new[src];
  }
}

static int copy_grid(long long pieces) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (pieces + 255) / 256;
  const long long cap = static_cast<long long>(sms > 0 ? sms : 1) * 8;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

int launch_ring_linearize(const void* ring_k, const void* ring_v, const void* k_new, const void* v_new, void* k_lin,
                          void* v_lin, int S, int T, int delta, int past, int slots, cudaStream_t st) {
  if (S <= 0 || T <= 0) return (S == 0 || T == 0) ? 0 : -1;
  if (slots <= 0 || delta < 0 || delta > past || delta >= slots + 1) return -1;
  if ((reinterpret_cast<uintptr_t>(ring_k) | reinterpret_cast<uintptr_t>(ring_v) | reinterpret_cast<uintptr_t>(k_new) |
       reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(k_lin) | reinterpret_cast<uintptr_t>(v_lin)) & 15u)
    return -3;
  const long long pieces = static_cast<long long>(S) * (delta + T) * 64;
  ring_linearize_kernel<<<copy_grid(pieces), 256, 0, st>>>(
      static_cast<const uint4*>(ring_k), static_cast<const uint4*>(ring_v), static_cast<const uint4*>(k_new),
      static_cast<const uint4*>(v_new), static_cast<uint4*>(k_lin), static_cast<uint4*>(v_lin), S, T, delta, past, slots);
  return static_cast<int>(cudaGetLastError());
}

int launch_ring_append(const void* k_new, const void* v_new, void* ring_k, void* ring_v, int S, int T, int past,
                       int slots, cudaStream_t st) {
  if (S <= 0 || T <= 0) return (S == 0 || T == 0) ? 0 : -1;
  if (slots <= 0 || past < 0) return -1;
  if ((reinterpret_cast<uintptr_t>(ring_k) | reinterpret_cast<uintptr_t>(ring_v) | reinterpret_cast<uintptr_t>(k_new) |
       reinterpret_cast<uintptr_t>(v_new)) & 15u)
    return -3;
  const int t_first = T > slots ? T - slots : 0;
  const long long pieces = static_cast<long long>(S) * (T - t_first) * 64;
  ring_append_kernel<<<copy_grid(pieces), 256, 0, st>>>(static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new),
                                                        static_cast<uint4*>(ring_k), static_cast<uint4*>(ring_v), S, T,
                                                        t_first, past, slots);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
