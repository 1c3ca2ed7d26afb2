// LayerNorm over the 512-wide hidden dimension, written for the activations that feed the tensor-core
// projections: input in FP32, FP16 or BF16, output rounded once to FP16 or BF16.
//
// Replaces nn.LayerNorm(hidden_size, eps) in front of the attention and MLP branches of the reference's
// transformer layer (src/fast_mimi/model.py:2021-2024, applied at :2052 and :2060): biased variance,
// (x - mean) * rsqrt(var + eps) * weight + bias, all in FP32.
//
// One warp per frame: each lane holds 16 values (four 4-element pieces, 32 lanes apart, so every load and
// store instruction of the warp touches one contiguous run), two shuffle reductions, no shared memory.
// HBM-bound: reads the frame once, writes it once.
#include <type_traits>

#include "fm_common.cuh"
#include "fm_kernels.h"

namespace fm {

namespace ln {
constexpr int kHidden = 512;
constexpr int kWarpsPerBlock = 8;

template <int kIn>
__device__ __forceinline__ void load4(const void* base, long long elem, float (&v)[4]) {
  if constexpr (kIn == 2) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem));
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  } else {
    using T16 = typename std::conditional<kIn == 1, __half, __nv_bfloat16>::type;
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + elem));
    const float2 a = Pack16<T16>::unpack(u.x), b = Pack16<T16>::unpack(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
}  // namespace ln

// kIn: 0 = BF16, 1 = FP16, 2 = FP32;  kOut: 0 = BF16, 1 = FP16
template <int kIn, int kOut>
__global__ void __launch_bounds__(ln::kWarpsPerBlock * 32)
layernorm512_kernel(const void* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ bias,
                    float eps, void* __restrict__ y, long long rows) {
  using namespace ln;
  using TOut = typename std::conditional<kOut == 1, __half, __nv_bfloat16>::type;
  const int lane = threadIdx.x & 31;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * kWarpsPerBlock;
  // this lane's channels: 4*lane + 128*j + (0..3); weight and bias stay in registers across frames
  float w[4][4], b[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 wf = __ldg(reinterpret_cast<const float4*>(weight + 128 * j + 4 * lane));
    const float4 bf = __ldg(reinterpret_cast<const float4*>(bias + 128 * j + 4 * lane));
    w[j][0] = wf.x; w[j][1] = wf.y; w[j][2] = wf.z; w[j][3] = wf.w;
    b[j][0] = bf.x; b[j][1] = bf.y; b[j][2] = bf.z; b[j][3] = bf.w;
  }
  for (long long row = warp0; row < rows; row += stride) {
    float v[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) load4<kIn>(x, row * kHidden + 128 * j + 4 * lane, v[j]);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) sum += (v[j][0] + v[j][1]) + (v[j][2] + v[j][3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum * (1.0f / kHidden);
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[j][e] -= mean;
        sq += v[j][e] * v[j][e];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq * (1.0f / kHidden) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = v[j][e] * rstd * w[j][e] + b[j][e];
      const uint2 packed = make_uint2(Pack16<TOut>::pack(o[0], o[1]), Pack16<TOut>::pack(o[2], o[3]));
      *reinterpret_cast<uint2*>(static_cast<uint16_t*>(y) + row * kHidden + 128 * j + 4 * lane) = packed;
    }
  }
}

int launch_layernorm512(const void* x, int x_dtype, const float* weight, const float* bias, float eps, void* y,
                        int y_dtype, long long rows, cudaStream_t st) {
  using namespace ln;
  if (rows < 0 || x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 1) return -1;
  if (rows == 0) return 0;
  if (x == nullptr || y == nullptr || weight == nullptr || bias == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(bias)) & 15u)
    return -3;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = static_cast<long long>(sms > 0 ? sms : 1) * 8;    // 8 resident blocks of 256 threads per SM
  const int grid = static_cast<int>(want < cap ? want : cap);
  using Kern = void (*)(const void*, const float*, const float*, float, void*, long long);
  static const Kern table[3][2] = {{layernorm512_kernel<0, 0>, layernorm512_kernel<0, 1>},
                                   {layernorm512_kernel<1, 0>, layernorm512_kernel<1, 1>},
                                   {layernorm512_kernel<2, 0>, layernorm512_kernel<2, 1>}};
  table[x_dtype][y_dtype]<<<grid, kWarpsPerBlock * 32, 0, st>>>(x, weight, bias, eps, y, rows);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fm
