// The two stride-2 convolutions around the quantiser (sm_100a): `downsample` after the encoder transformer and
// `upsample` before the decoder transformer.
//
// Downsample.
// Reference: MimiModel.downsample = MimiConv1d(512 -> 512, kernel 4, stride 2, no bias, replicate padding, causal)
// (src/fast_mimi/model.py:2734-2744; forward of the class: left padding kernel - stride = 2 frames, right padding
// (-T) % 2 frames, both repeating the edge frame, then nn.Conv1d).  On frame-major activations [B, T, 512] output
// frame t is a 2048-long inner product: the four consecutive frames 2t-2 .. 2t+1 (clamped to the clip) against
// the kernel laid out as W2[c_out, j * 512 + c_in] = W[c_out, c_in, j].  So the convolution is a linear with
// K = 2048 over rows that overlap in memory; this file only gathers those rows (with the edge clamping) and splits
// them into FP16 hi + lo parts; the products run on the tensor-core linear kernel (hi W_hi + hi W_lo + lo W_hi with
// FP32 accumulation: FP32-grade accuracy, which the code decisions that follow need).
#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

// One thread per 8 values of a gathered row: rows [B * T_out, 4 * C], x [B, T, C] FP32 (C a multiple of 8).
__global__ void __launch_bounds__(256)
conv_rows_split_kernel(const float* __restrict__ x, uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, int B, int T,
                       int T_out, int C, int kernel, int stride) {
  const int c8 = C / 8;
  const long long total = static_cast<long long>(B) * T_out * kernel * c8;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int piece = static_cast<int>(i % c8);
    long long r = i / c8;
    const int j = static_cast<int>(r % kernel);
    r /= kernel;
    const int t = static_cast<int>(r % T_out);
    const long long b = r / T_out;
    int f = t * stride + j - (kernel - stride);          // frame of the padded sequence, replicate at both ends
    f = f < 0 ? 0 : (f > T - 1 ? T - 1 : f);
    const float4* src = reinterpret_cast<const float4*>(x + (b * T + f) * C + piece * 8);
    const float4 a = __ldg(src), c = __ldg(src + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
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

int launch_conv_rows_split(const float* x, void* hi, void* lo, int B, int T, int C, int kernel, int stride,
                           cudaStream_t st) {
  if (B <= 0 || T <= 0) return (B == 0 || T == 0) ? 0 : -1;
  if (C <= 0 || C % 8 != 0 || kernel < stride || stride <= 0 || kernel > 16) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15u) return -3;
  const int T_out = (T + stride - 1) / stride;
  const long long total = static_cast<long long>(B) * T_out * kernel * (C / 8);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (total + 255) / 256, cap = static_cast<long long>(sms > 0 ? sms : 1) * 8;
  conv_rows_split_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, st>>>(
      x, static_cast<uint16_t*>(hi), static_cast<uint16_t*>(lo), B, T, T_out, C, kernel, stride);
  return static_cast<int>(cudaGetLastError());
}

// Upsample.  Reference: MimiModel.upsample = MimiConvTranspose1d(512 -> 512, kernel 4, stride 2, groups = 512, no bias)
// (src/fast_mimi/model.py:2745-2753; forward of the class: nn.ConvTranspose1d, then the last kernel - stride = 2
// output frames are trimmed, causal with trim_right_ratio 1).  With one channel per group it is elementwise: on
// frame-major activations  y[b, n, c] = w[c, n % 2] x[b, n / 2, c] + w[c, n % 2 + 2] x[b, n / 2 - 1, c]  for
// n = 0 .. 2T-1 (the second term absent for n < 2).  FP32 in, FP32 out, HBM-bound: 4 bytes read (each x value serves
// four outputs through L1 / L2) and 8 written per input value.
__global__ void __launch_bounds__(256)
upsample2_depthwise_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int B, int T,
                           int C) {
  const int c4 = C / 4;
  const long long total = static_cast<long long>(B) * 2 * T * c4;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int cq = static_cast<int>(i % c4);
    long long r = i / c4;
    const int n = static_cast<int>(r % (2 * T));
    const long long b = r / (2 * T);
    const int t = n >> 1, j = n & 1;
    const float4 a = __ldg(reinterpret_cast<const float4*>(x + (b * T + t) * C) + cq);
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t > 0) p = __ldg(reinterpret_cast<const float4*>(x + (b * T + t - 1) * C) + cq);
    const float* wc = w + static_cast<long long>(cq) * 16;        // four channels x four taps
    float4 o;
    o.x = wc[j] * a.x + wc[j + 2] * p.x;
    o.y = wc[4 + j] * a.y + wc[4 + j + 2] * p.y;
    o.z = wc[8 + j] * a.z + wc[8 + j + 2] * p.z;
    o.w = wc[12 + j] * a.w + wc[12 + j + 2] * p.w;
    reinterpret_cast<float4*>(y + (b * 2 * T + n) * C)[cq] = o;
  }
}

int launch_upsample2_depthwise(const float* x, const float* w, float* y, int B, int T, int C, cudaStream_t st) {
  if (B <= 0 || T <= 0) return (B == 0 || T == 0) ? 0 : -1;
  if (C <= 0 || C % 4 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15u) return -3;
  const long long total = static_cast<long long>(B) * 2 * T * (C / 4);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (total + 255) / 256, cap = static_cast<long long>(sms > 0 ? sms : 1) * 8;
  upsample2_depthwise_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, st>>>(x, w, y, B, T, C);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
