// FP32 verification kernels (CUDA cores, no tensor cores): a generic restatement of the
// attention path used to check the tensor-core kernels and to run small / odd geometries
// (any head count, head_dim <= 256, any window, cached chunks with position offsets).
//
// Reference semantics followed (paths relative to the reference project):
//   projections   src/fast_mimi/model.py:1897-1911   y = x W^T, no bias
//   RoPE          src/fast_mimi/model.py:1538-1569   x*cos + rotate_half(x)*sin
//   band mask     src/fast_mimi/model.py:1672-1676   qpos-window < kpos <= qpos
//   attention     src/fast_mimi/model.py:1953-1958   softmax(scale*q.k + mask) v, FP32
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

// y[m, n] = sum_k x[m, k] * w[n, k]; one thread per output, sequential FP32 FMA.
__global__ void linear_fp32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   float* __restrict__ y, int M, int N, int K) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(M) * N) return;
  const int m = static_cast<int>(idx / N), n = static_cast<int>(idx % N);
  const float* xr = x + static_cast<long long>(m) * K;
  const float* wr = w + static_cast<long long>(n) * K;
  float acc = 0.f;
  for (int k = 0; k < K; ++k) acc = fmaf(xr[k], wr[k], acc);
  y[idx] = acc;
}

// In-place rotate-half RoPE on t[B, T, H, D] (row stride H*D); cos/sin are [Bc, T, D] with
// batch stride cos_bstride (0 broadcasts one table over the batch).
__global__ void rope_fp32_kernel(float* __restrict__ t, const float* __restrict__ cosv,
                                 const float* __restrict__ sinv, int B, int T, int H, int D,
                                 long long cos_bstride) {
  const int half = D / 2;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total = static_cast<long long>(B) * T * H * half;
  if (idx >= total) return;
  const int d = static_cast<int>(idx % half);
  const int h = static_cast<int>((idx / half) % H);
  const int tt = static_cast<int>((idx / (static_cast<long long>(half) * H)) % T);
  const int b = static_cast<int>(idx / (static_cast<long long>(half) * H * T));
  float* p = t + ((static_cast<long long>(b) * T + tt) * H + h) * D;
  const float* c = cosv + b * cos_bstride + static_cast<long long>(tt) * D;
  const float* s = sinv + b * cos_bstride + static_cast<long long>(tt) * D;
  const float lo = p[d], hi = p[d + half];
  // Separate multiplies and adds, as the reference's unfused tensor expression evaluates them.
  p[d] = __fadd_rn(__fmul_rn(lo, c[d]), __fmul_rn(-hi, s[d]));
  p[d + half] = __fadd_rn(__fmul_rn(hi, c[d + half]), __fmul_rn(lo, s[d + half]));
}

// One warp per (batch, head, query row).  Two passes over the visible keys: row maximum,
// then exp / sum / weighted V accumulation, all FP32 with warp-shuffle reductions.
// Strides are in elements; the last dimension (head_dim) is contiguous.
__global__ void band_attn_fp32_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                      const float* __restrict__ v, float* __restrict__ out, int B, int H,
                                      int D, int Tq, int Tk, int q_off, int k_off, int window, float scale,
                                      long long qs_b, long long qs_h, long long qs_t, long long ks_b,
                                      long long ks_h, long long ks_t, long long vs_b, long long vs_h,
                                      long long vs_t, long long os_b, long long os_h, long long os_t) {
  constexpr int kMaxPerLane = 8;  // head_dim <= 256
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (warp >= static_cast<long long>(B) * H * Tq) return;
  const int i = static_cast<int>(warp % Tq);
  const int h = static_cast<int>((warp / Tq) % H);
  const int b = static_cast<int>(warp / (static_cast<long long>(Tq) * H));
  const float* qp = q + b * qs_b + h * qs_h + i * qs_t;
  float qreg[kMaxPerLane];
#pragma unroll
  for (int r = 0; r < kMaxPerLane; ++r) {
    const int d = lane + 32 * r;
    qreg[r] = d < D ? qp[d] : 0.f;
  }
  // Visible keys: absolute position in (qpos - window, qpos], index = position - k_off.
  const int qpos = i + q_off;
  int j_lo = qpos - window + 1 - k_off;
  int j_hi = qpos - k_off;
  if (j_lo < 0) j_lo = 0;
  if (j_hi > Tk - 1) j_hi = Tk - 1;
  const float* kb = k + b * ks_b + h * ks_h;
  const float* vb = v + b * vs_b + h * vs_h;

  float m = -INFINITY;
  for (int j = j_lo; j <= j_hi; ++j) {
    const float* kp = kb + j * ks_t;
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
      const int d = lane + 32 * r;
      if (d < D) part = fmaf(qreg[r], kp[d], part);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    m = fmaxf(m, part * scale);
  }
  float l = 0.f;
  float acc[kMaxPerLane];
#pragma unroll
  for (int r = 0; r < kMaxPerLane; ++r) acc[r] = 0.f;
  for (int j = j_lo; j <= j_hi; ++j) {
    const float* kp = kb + j * ks_t;
    const float* vp = vb + j * vs_t;
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
      const int d = lane + 32 * r;
      if (d < D) part = fmaf(qreg[r], kp[d], part);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float p = expf(part * scale - m);
    l += p;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
      const int d = lane + 32 * r;
      if (d < D) acc[r] = fmaf(p, vp[d], acc[r]);
    }
  }
  float* op = out + b * os_b + h * os_h + i * os_t;
  const float inv = (j_hi >= j_lo) ? 1.f / l : 0.f;
#pragma unroll
  for (int r = 0; r < kMaxPerLane; ++r) {
    const int d = lane + 32 * r;
    if (d < D) op[d] = acc[r] * inv;
  }
}

int launch_linear_fp32(const float* x, const float* w, float* y, int M, int N, int K, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return M == 0 || N == 0 ? 0 : -1;
  const long long total = static_cast<long long>(M) * N;
  linear_fp32_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(x, w, y, M, N, K);
  return static_cast<int>(cudaGetLastError());
}

int launch_rope_fp32(float* t, const float* cosv, const float* sinv, int B, int T, int H, int D,
                     long long cos_bstride, cudaStream_t st) {
  if (D <= 0 || (D & 1)) return -1;
  const long long total = static_cast<long long>(B) * T * H * (D / 2);
  if (total == 0) return 0;
  rope_fp32_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(t, cosv, sinv, B, T, H, D,
                                                                              cos_bstride);
  return static_cast<int>(cudaGetLastError());
}

int launch_band_attn_fp32(const float* q, const float* k, const float* v, float* out, int B, int H, int D,
                          int Tq, int Tk, int q_off, int k_off, int window, float scale,
                          const long long* strides, cudaStream_t st) {
  if (D <= 0 || D > 256 || window <= 0 || B < 0 || H <= 0 || Tq < 0 || Tk < 0) return -1;
  const long long warps = static_cast<long long>(B) * H * Tq;
  if (warps == 0) return 0;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return -2;
  band_attn_fp32_kernel<<<static_cast<unsigned>(blocks), threads, 0, st>>>(
      q, k, v, out, B, H, D, Tq, Tk, q_off, k_off, window, scale, strides[0], strides[1], strides[2],
      strides[3], strides[4], strides[5], strides[6], strides[7], strides[8], strides[9], strides[10],
      strides[11]);
  return static_cast<int>(cudaGetLastError());
}

// Self-test of the bounded-wait machinery: one thread waits on a barrier that nothing ever arrives on, with a
// limit of `limit_us` microseconds; the wait gives up, records kErrWaitConsumer in the status word and the kernel
// returns normally (no trap, no unbounded loop).  A second wait in the same CTA returns at once (abort flag).
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns, int* observed) {
  __shared__ uint64_t bar;
  __shared__ CtaCtl ctl;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    ctl.abort = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool first = mbar_wait_limit(&bar, 0, &ctl, status, kErrWaitConsumer, limit_ns);
    const unsigned long long t0 = global_timer_ns();
    const bool second = mbar_wait_limit(&bar, 0, &ctl, status, kErrWaitTma, limit_ns);
    const unsigned long long dt = global_timer_ns() - t0;
    if (observed != nullptr) {
      observed[0] = first ? 1 : 0;
      observed[1] = second ? 1 : 0;
      observed[2] = dt < limit_ns ? 1 : 0;       // the second wait did not sit out the limit again
    }
  }
}

int launch_wait_timeout_selftest(int* status, int limit_us, int* observed, cudaStream_t st) {
  if (status == nullptr || limit_us <= 0 || limit_us > 100000) return -1;
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(status, static_cast<unsigned long long>(limit_us) * 1000ull, observed);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
