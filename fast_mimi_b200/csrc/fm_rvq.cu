// Residual vector quantisation around the encoder transformer (sm_100a): nearest-codebook search and ordered
// decode for Mimi's Euclidean codebooks (2048 entries of 256 dimensions per layer).
//
// Reference: MimiEuclideanCodebook.quantize = argmin over torch.cdist (src/fast_mimi/model.py:2277-2291),
// MimiResidualVectorQuantizer.encode subtracts the chosen entry before the next layer's search
// (src/fast_mimi/model.py:2408-2429), decode adds the layers' entries left to right starting from an FP32 zero
// (src/fast_mimi/model.py:2431-2444).
//
// Search: the 2048 inner products per frame are a GEMM and run on the tensor core with FP16 operands (the general
// linear kernel of this library, K = 256, N = 2048).  They only PRE-SELECT: for a frame x the approximate
// distances  |e_j|^2 - 2 x.e_j  differ from the exact ones by at most  tau = tau_rel * |x| * max_j |e_j|
// (see the derivation of tau_rel below), so
// every entry within tau of the approximate minimum is a candidate and the entry that wins is decided among the
// candidates by the exact FP32 distance
// sum_k (x_k - e_jk)^2, lowest index on ties (argmin's rule).  rvq_select_kernel does that per frame with one
// warp, writes the code, subtracts the entry from the residual (FP32, in place) and emits the FP16 copy of the
// new residual that the next layer's GEMM consumes.
//
// tau_rel: rounding x and e to FP16 perturbs x.e by at most 2 * 2^-11 |x||e| (to first order), storing the score as
// FP16 by another 2^-11 |x||e|, so d_j = |e_j|^2 - 2 x.e_j is off by at most 4 * 2^-11 |x||e| = 1.95e-3 |x||e| with
// FP32 scores and 6 * 2^-11 |x||e| = 2.93e-3 |x||e| with FP16 scores.  The true winner's d may be too high and the
// approximate minimum too low by that much each, so the candidate margin must be twice the bound: 3.9e-3 and
// 5.86e-3.  Callers pass 4.5e-3 / 6.0e-3.
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace rvq {
constexpr int kDim = 256;        // codebook dimension
constexpr int kWarps = 8;        // warps (frames in flight) per block
constexpr int kMaxIters = 16;    // a lane keeps 4 * kMaxIters approximate distances: up to 2048 entries per codebook

// Four consecutive scores of a row, stored as FP32 or as FP16.
template <bool kHalf>
__device__ __forceinline__ float4 load_scores4(const void* row_base, int v) {
  if constexpr (kHalf) {
    const uint2 u = reinterpret_cast<const uint2*>(row_base)[v];
    const float2 a = Pack16<__half>::unpack(u.x), b = Pack16<__half>::unpack(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  } else {
    return reinterpret_cast<const float4*>(row_base)[v];
  }
}
}  // namespace rvq

template <bool kHalf>
__global__ void __launch_bounds__(rvq::kWarps * 32)
rvq_select_kernel(const void* __restrict__ scores, const float* __restrict__ e_sq, const float* __restrict__ codebook,
                  float* __restrict__ resid, uint16_t* __restrict__ resid16, long long* __restrict__ codes,
                  int* __restrict__ n_candidates, long long rows, int n_codes, float e_max, float tau_rel,
                  int* __restrict__ status) {
  using namespace rvq;
  const int lane = threadIdx.x & 31;
  const int n_iters = n_codes >> 7;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * kWarps;
  for (long long row = warp0; row < rows; row += stride) {
    // this lane's 8 residual values (dimensions 8 * lane .. 8 * lane + 7)
    float x[8];
    {
      const float4* xr = reinterpret_cast<const float4*>(resid + row * kDim + lane * 8);
      const float4 a = xr[0], b = xr[1];
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    float xx = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) xx = fmaf(x[k], x[k], xx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) xx += __shfl_xor_sync(0xffffffffu, xx, o);
    // relative part: FP16 rounding of both operands; absolute part: residual values below FP16's normal range
    const float tau = tau_rel * sqrtf(xx) * e_max + 3.1e-5f * e_max;      // == rvq_margin below

    // pass A: approximate distances of this lane's entries (kept in registers) and their minimum.  Lane l holds
    // entries 128 * it + 4 * l + e, it = 0 .. n_codes / 128 - 1, e = 0 .. 3.
    const void* s4 = static_cast<const uint8_t*>(scores) + static_cast<size_t>(row) * n_codes * (kHalf ? 2 : 4);
    const float4* q4 = reinterpret_cast<const float4*>(e_sq);
    float d[kMaxIters][4];
    float d_min = INFINITY;
#pragma unroll
    for (int it = 0; it < kMaxIters; ++it) {
      if (it < n_iters) {                            // the same for every lane
        const float4 s = load_scores4<kHalf>(s4, it * 32 + lane), q = __ldg(q4 + it * 32 + lane);
        d[it][0] = fmaf(-2.f, s.x, q.x); d[it][1] = fmaf(-2.f, s.y, q.y);
        d[it][2] = fmaf(-2.f, s.z, q.z); d[it][3] = fmaf(-2.f, s.w, q.w);
        d_min = fminf(d_min, fminf(fminf(d[it][0], d[it][1]), fminf(d[it][2], d[it][3])));
      } else {
        d[it][0] = d[it][1] = d[it][2] = d[it][3] = INFINITY;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d_min = fminf(d_min, __shfl_xor_sync(0xffffffffu, d_min, o));
    const float limit = d_min + tau;

    // pass B: every lane marks its candidates (bit 4 * it + e); the warp then evaluates them one by one exactly
    unsigned long long mine = 0ull;
#pragma unroll
    for (int it = 0; it < kMaxIters; ++it) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (d[it][e] <= limit) mine |= 1ull << (4 * it + e);
    }
    float best = INFINITY;
    int best_j = 0, n_cand = 0;
    unsigned lanes = __ballot_sync(0xffffffffu, mine != 0ull);
    while (lanes != 0u) {
      const int src = __ffs(lanes) - 1;
      lanes &= lanes - 1u;
      unsigned long long bits = __shfl_sync(0xffffffffu, mine, src);
      while (bits != 0ull) {
        const int bit = __ffsll(static_cast<long long>(bits)) - 1;
        bits &= bits - 1ull;
        const int j = (bit >> 2) * 128 + src * 4 + (bit & 3);
        const float4* er = reinterpret_cast<const float4*>(codebook + static_cast<size_t>(j) * kDim + lane * 8);
        const float4 a = __ldg(er), b = __ldg(er + 1);
        const float ev[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float t = x[k] - ev[k];
          acc = fmaf(t, t, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        ++n_cand;
        // candidates do not come in index order: ties go to the lower index explicitly (argmin's rule)
        if (acc < best || (acc == best && j < best_j)) {
          best = acc;
          best_j = j;
        }
      }
    }

    // the chosen entry leaves the residual; the next layer's GEMM reads the FP16 copy
    {
      const float4* er = reinterpret_cast<const float4*>(codebook + static_cast<size_t>(best_j) * kDim + lane * 8);
      const float4 a = __ldg(er), b = __ldg(er + 1);
      const float ev[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] -= ev[k];
      float4* xw = reinterpret_cast<float4*>(resid + row * kDim + lane * 8);
      xw[0] = make_float4(x[0], x[1], x[2], x[3]);
      xw[1] = make_float4(x[4], x[5], x[6], x[7]);
      *reinterpret_cast<uint4*>(resid16 + row * kDim + lane * 8) =
          make_uint4(Pack16<__half>::pack(x[0], x[1]), Pack16<__half>::pack(x[2], x[3]), Pack16<__half>::pack(x[4], x[5]),
                     Pack16<__half>::pack(x[6], x[7]));
    }
    if (lane == 0) {
      codes[row] = best_j;
      if (n_candidates != nullptr) n_candidates[row] = n_cand;
      // A residual that is not finite (or overflows FP16) makes every approximate distance NaN: nothing was a
      // candidate and the code above is meaningless.  Say so instead of emitting entry 0 silently.
      if (n_cand == 0 && status != nullptr) atomicMax(status, static_cast<int>(kErrNonFinite));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same search without the scores' round trip through memory: the inner-product GEMM's epilogue (linear kernel,
// record mode) reduces every 64 entries of a frame to one 16-byte record {minimum approximate distance, 64-bit mask of
// the entries within the frame's margin of that minimum}, 32 records per frame for 2048 entries (512 B instead of
// 4 KB of FP16 scores).  An entry within the margin of the GLOBAL minimum is within the margin of its own group's
// minimum, so the union of the masks of the groups whose minimum is within the margin of the global one contains every
// true candidate; the extra ones only cost an exact evaluation each.  The margin of a frame depends on its residual
// norm, which the previous layer's decision kernel (or rvq_prepare_kernel before the first layer) leaves in `tau`.
__device__ __forceinline__ float rvq_margin(float xx, float e_max, float tau_rel) {
  // relative part: FP16 rounding of both operands; absolute part: residual values below FP16's normal range
  return tau_rel * sqrtf(xx) * e_max + 3.1e-5f * e_max;
}

__global__ void __launch_bounds__(rvq::kWarps * 32)
rvq_select_rec_kernel(const uint4* __restrict__ records, const float* __restrict__ codebook, float* __restrict__ resid,
                      uint16_t* __restrict__ resid16, long long* __restrict__ codes, int* __restrict__ n_candidates,
                      float* __restrict__ tau, long long rows, int n_groups, float e_max_next, float tau_rel,
                      int* __restrict__ status) {
  using namespace rvq;
  const int lane = threadIdx.x & 31;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * kWarps;
  for (long long row = warp0; row < rows; row += stride) {
    float x[8];
    {
      const float4* xr = reinterpret_cast<const float4*>(resid + row * kDim + lane * 8);
      const float4 a = xr[0], b = xr[1];
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    // this lane's group (entries 64 * lane .. 64 * lane + 63): its minimum and its mask
    uint4 rec = make_uint4(__float_as_uint(INFINITY), 0u, 0u, 0u);
    if (lane < n_groups) rec = records[row * n_groups + lane];
    const float gmin = __uint_as_float(rec.x);
    float d_min = gmin;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d_min = fminf(d_min, __shfl_xor_sync(0xffffffffu, d_min, o));
    const float limit = d_min + tau[row];
    unsigned long long mine = gmin <= limit ? (static_cast<unsigned long long>(rec.z) << 32) | rec.y : 0ull;

    float best = INFINITY;
    int best_j = 0, n_cand = 0;
    unsigned lanes = __ballot_sync(0xffffffffu, mine != 0ull);
    while (lanes != 0u) {
      const int src = __ffs(lanes) - 1;
      lanes &= lanes - 1u;
      unsigned long long bits = __shfl_sync(0xffffffffu, mine, src);
      while (bits != 0ull) {
        const int bit = __ffsll(static_cast<long long>(bits)) - 1;
        bits &= bits - 1ull;
        const int j = src * 64 + bit;
        const float4* er = reinterpret_cast<const float4*>(codebook + static_cast<size_t>(j) * kDim + lane * 8);
        const float4 a = __ldg(er), b = __ldg(er + 1);
        const float ev[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float t = x[k] - ev[k];
          acc = fmaf(t, t, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        ++n_cand;
        if (acc < best || (acc == best && j < best_j)) {      // ties go to the lower index (argmin's rule)
          best = acc;
          best_j = j;
        }
      }
    }
    {
      const float4* er = reinterpret_cast<const float4*>(codebook + static_cast<size_t>(best_j) * kDim + lane * 8);
      const float4 a = __ldg(er), b = __ldg(er + 1);
      const float ev[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      float xx = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        x[k] -= ev[k];
        xx = fmaf(x[k], x[k], xx);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) xx += __shfl_xor_sync(0xffffffffu, xx, o);
      float4* xw = reinterpret_cast<float4*>(resid + row * kDim + lane * 8);
      xw[0] = make_float4(x[0], x[1], x[2], x[3]);
      xw[1] = make_float4(x[4], x[5], x[6], x[7]);
      *reinterpret_cast<uint4*>(resid16 + row * kDim + lane * 8) =
          make_uint4(Pack16<__half>::pack(x[0], x[1]), Pack16<__half>::pack(x[2], x[3]), Pack16<__half>::pack(x[4], x[5]),
                     Pack16<__half>::pack(x[6], x[7]));
      if (lane == 0) tau[row] = rvq_margin(xx, e_max_next, tau_rel);      // the next layer's margin for this frame
    }
    if (lane == 0) {
      codes[row] = best_j;
      if (n_candidates != nullptr) n_candidates[row] = n_cand;
      if (n_cand == 0 && status != nullptr) atomicMax(status, static_cast<int>(kErrNonFinite));
    }
  }
}

// Before the first layer: FP16 copy of the residual and every frame's candidate margin (one warp per frame).
__global__ void __launch_bounds__(rvq::kWarps * 32)
rvq_prepare_kernel(const float* __restrict__ x, uint16_t* __restrict__ resid16, float* __restrict__ tau, long long rows,
                   float e_max, float tau_rel) {
  using namespace rvq;
  const int lane = threadIdx.x & 31;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * kWarps;
  for (long long row = warp0; row < rows; row += stride) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * kDim + lane * 8);
    const float4 a = xr[0], b = xr[1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float xx = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) xx = fmaf(v[k], v[k], xx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) xx += __shfl_xor_sync(0xffffffffu, xx, o);
    *reinterpret_cast<uint4*>(resid16 + row * kDim + lane * 8) =
        make_uint4(Pack16<__half>::pack(v[0], v[1]), Pack16<__half>::pack(v[2], v[3]), Pack16<__half>::pack(v[4], v[5]),
                   Pack16<__half>::pack(v[6], v[7]));
    if (lane == 0) tau[row] = rvq_margin(xx, e_max, tau_rel);
  }
}

// FP32 -> FP16 copy of the residual before the first layer (256 values per frame).
__global__ void __launch_bounds__(256)
rvq_to_half_kernel(const float* __restrict__ x, uint16_t* __restrict__ y, long long n8) {
  const long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = i0; i < n8; i += stride) {
    const float4 a = reinterpret_cast<const float4*>(x)[2 * i], b = reinterpret_cast<const float4*>(x)[2 * i + 1];
    reinterpret_cast<uint4*>(y)[i] = make_uint4(Pack16<__half>::pack(a.x, a.y), Pack16<__half>::pack(a.z, a.w),
                                                Pack16<__half>::pack(b.x, b.y), Pack16<__half>::pack(b.z, b.w));
  }
}

// x = hi + lo with both parts in FP16 (hi = round(x), lo = round(x - hi)): 22 significant bits, enough for an
// FP32-grade product on the FP16 tensor core as  hi W_hi + hi W_lo + lo W_hi  with FP32 accumulation.
__global__ void __launch_bounds__(256)
split_half_kernel(const float* __restrict__ x, uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, long long n8) {
  const long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = i0; i < n8; i += stride) {
    const float4 a = reinterpret_cast<const float4*>(x)[2 * i], b = reinterpret_cast<const float4*>(x)[2 * i + 1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = Pack16<__half>::pack(v[2 * e], v[2 * e + 1]);
      const float2 back = Pack16<__half>::unpack(h[e]);
      l[e] = Pack16<__half>::pack(v[2 * e] - back.x, v[2 * e + 1] - back.y);
    }
    reinterpret_cast<uint4*>(hi)[i] = make_uint4(h[0], h[1], h[2], h[3]);
    reinterpret_cast<uint4*>(lo)[i] = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// out[row, :] = ((0 + E_0[c_0]) + E_1[c_1]) + ...  in FP32, layers left to right.
__global__ void __launch_bounds__(256)
rvq_decode_kernel(const long long* __restrict__ codes, const float* __restrict__ codebooks, float* __restrict__ out,
                  long long rows, int n_layers, int n_codes, int* __restrict__ bad_code) {
  using namespace rvq;
  const int sub = threadIdx.x & 63;                 // 64 threads per frame, 4 dimensions each
  const long long row0 = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 6);
  const long long stride = static_cast<long long>(gridDim.x) * 4;
  for (long long row = row0; row < rows; row += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int l = 0; l < n_layers; ++l) {
      long long cidx = codes[static_cast<long long>(l) * rows + row];
      if (cidx < 0 || cidx >= n_codes) {            // recorded, not dereferenced
        if (bad_code != nullptr) atomicExch(bad_code, 1);
        cidx = 0;
      }
      const float4 e = __ldg(reinterpret_cast<const float4*>(
          codebooks + (static_cast<size_t>(l) * n_codes + static_cast<size_t>(cidx)) * kDim + sub * 4));
      acc.x += e.x; acc.y += e.y; acc.z += e.z; acc.w += e.w;
    }
    reinterpret_cast<float4*>(out + row * kDim)[sub] = acc;
  }
}

static int grid_for(long long work_blocks, int per_sm) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long cap = static_cast<long long>(sms > 0 ? sms : 1) * per_sm;
  const long long g = work_blocks < cap ? work_blocks : cap;
  return static_cast<int>(g > 0 ? g : 1);
}

int launch_rvq_select(const void* scores, int scores_fp16, const float* e_sq, const float* codebook, float* resid, void* resid16,
                      long long* codes, int* n_candidates, long long rows, int n_codes, float e_max, float tau_rel,
                      int* status, cudaStream_t st) {
  if (rows < 0 || n_codes <= 0 || n_codes % 128 != 0 || n_codes > 128 * rvq::kMaxIters || !(e_max >= 0.f) ||
      !(tau_rel >= 0.f))
    return -1;
  if (rows == 0) return 0;
  if (scores == nullptr || e_sq == nullptr || codebook == nullptr || resid == nullptr || resid16 == nullptr || codes == nullptr)
    return -1;
  if ((reinterpret_cast<uintptr_t>(scores) | reinterpret_cast<uintptr_t>(e_sq) | reinterpret_cast<uintptr_t>(codebook) |
       reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(resid16)) & 15u)
    return -3;
  const int grid = grid_for((rows + rvq::kWarps - 1) / rvq::kWarps, 8);
  if (scores_fp16)
    rvq_select_kernel<true><<<grid, rvq::kWarps * 32, 0, st>>>(scores, e_sq, codebook, resid, static_cast<uint16_t*>(resid16),
                                                              codes, n_candidates, rows, n_codes, e_max, tau_rel, status);
  else
    rvq_select_kernel<false><<<grid, rvq::kWarps * 32, 0, st>>>(scores, e_sq, codebook, resid, static_cast<uint16_t*>(resid16),
                                                               codes, n_candidates, rows, n_codes, e_max, tau_rel, status);
  return static_cast<int>(cudaGetLastError());
}

int launch_rvq_select_rec(const void* records, const float* codebook, float* resid, void* resid16, long long* codes,
                          int* n_candidates, float* tau, long long rows, int n_codes, float e_max_next, float tau_rel,
                          int* status, cudaStream_t st) {
  if (rows < 0 || n_codes <= 0 || n_codes % 64 != 0 || n_codes > 2048 || !(e_max_next >= 0.f) || !(tau_rel >= 0.f)) return -1;
  if (rows == 0) return 0;
  if (records == nullptr || codebook == nullptr || resid == nullptr || resid16 == nullptr || codes == nullptr || tau == nullptr)
    return -1;
  if ((reinterpret_cast<uintptr_t>(records) | reinterpret_cast<uintptr_t>(codebook) | reinterpret_cast<uintptr_t>(resid) |
       reinterpret_cast<uintptr_t>(resid16)) & 15u)
    return -3;
  const int grid = grid_for((rows + rvq::kWarps - 1) / rvq::kWarps, 8);
  rvq_select_rec_kernel<<<grid, rvq::kWarps * 32, 0, st>>>(static_cast<const uint4*>(records), codebook, resid,
                                                          static_cast<uint16_t*>(resid16), codes, n_candidates, tau, rows,
                                                          n_codes / 64, e_max_next, tau_rel, status);
  return static_cast<int>(cudaGetLastError());
}

int launch_rvq_prepare(const float* x, void* resid16, float* tau, long long rows, float e_max, float tau_rel,
                       cudaStream_t st) {
  if (rows < 0 || !(e_max >= 0.f) || !(tau_rel >= 0.f)) return -1;
  if (rows == 0) return 0;
  if (x == nullptr || resid16 == nullptr || tau == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(resid16)) & 15u) return -3;
  rvq_prepare_kernel<<<grid_for((rows + rvq::kWarps - 1) / rvq::kWarps, 8), rvq::kWarps * 32, 0, st>>>(
      x, static_cast<uint16_t*>(resid16), tau, rows, e_max, tau_rel);
  return static_cast<int>(cudaGetLastError());
}

int launch_rvq_to_half(const float* x, void* y, long long rows, cudaStream_t st) {
  if (rows < 0) return -1;
  if (rows == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) return -3;
  const long long n8 = rows * (rvq::kDim / 8);
  rvq_to_half_kernel<<<grid_for((n8 + 255) / 256, 8), 256, 0, st>>>(x, static_cast<uint16_t*>(y), n8);
  return static_cast<int>(cudaGetLastError());
}

int launch_split_half(const float* x, void* hi, void* lo, long long n, cudaStream_t st) {
  if (n < 0 || n % 8 != 0) return -1;
  if (n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15u) return -3;
  const long long n8 = n / 8;
  split_half_kernel<<<grid_for((n8 + 255) / 256, 8), 256, 0, st>>>(x, static_cast<uint16_t*>(hi), static_cast<uint16_t*>(lo), n8);
  return static_cast<int>(cudaGetLastError());
}

int launch_rvq_decode(const long long* codes, const float* codebooks, float* out, long long rows, int n_layers, int n_codes,
                      int* bad_code, cudaStream_t st) {
  if (rows < 0 || n_layers <= 0 || n_codes <= 0) return -1;
  if (rows == 0) return 0;
  if (codes == nullptr || codebooks == nullptr || out == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(codebooks) | reinterpret_cast<uintptr_t>(out)) & 15u) return -3;
  rvq_decode_kernel<<<grid_for((rows + 3) / 4, 8), 256, 0, st>>>(codes, codebooks, out, rows, n_layers, n_codes, bad_code);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
