// extern "C" entry points of libfast_mimi_b200.so (declared in include/fast_mimi_b200.h) and the
// small host helpers they share.  No torch types, no allocation, no synchronisation except
// fm_read_status.
#include "../../include/fast_mimi_b200.h"

#include <mutex>

#include "fm_kernels.h"

namespace fm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, void* base, const cuuint64_t* dims,
                 const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* elem_strides,
                 CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -4;
  const CUresult r = fn(map, dtype, rank, base, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
  // cudaFuncSetAttribute is per device; remember the largest size granted to each (kernel, device) pair
  // and ask again only for more.
  constexpr int kMaxDev = 64, kMaxKern = 32;
  static std::mutex mu;
  static const void* kerns[kMaxKern];
  static int granted[kMaxKern][kMaxDev];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::lock_guard<std::mutex> lock(mu);
  int slot = -1;
  for (int i = 0; i < kMaxKern; ++i) {
    if (kerns[i] == kernel) { slot = i; break; }
    if (kerns[i] == nullptr) { kerns[i] = kernel; slot = i; break; }
  }
  if (slot >= 0 && dev < kMaxDev && granted[slot][dev] >= bytes) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (slot >= 0 && dev < kMaxDev) granted[slot][dev] = bytes;
  return 0;
}

}  // namespace fm

using fm::QkvEpilogueArgs;

extern "C" {

int fm_abi_version(void) { return 2; }

int fm_qkv_rope_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                     void* q, void* k, void* v, int B, int T, int value_dtype, int* status, void* stream) {
  if (B < 0 || T < 0 || value_dtype < 0 || value_dtype > 3) return -1;
  if (static_cast<long long>(B) * T > 0x7fffffffLL) return -1;
  QkvEpilogueArgs ep = {};
  ep.q = static_cast<uint16_t*>(q);
  ep.k = static_cast<uint16_t*>(k);
  ep.v = static_cast<uint16_t*>(v);
  ep.cos = cos;
  ep.sin = sin;
  ep.cos_bstride = cos_bstride;
  ep.T = T;
  ep.ring_slots = 1;
  return fm::launch_qkv_rope_gemm(x, w_qkv, ep, B * T, value_dtype, status, static_cast<cudaStream_t>(stream));
}

int fm_band_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, int B, int T, int window,
                              float scale, int value_dtype, int* status, void* stream) {
  if (value_dtype != 0 && value_dtype != 1) return -1;
  return fm::launch_band_attn_prefill(q, k, v, out, B, T, window, scale, value_dtype, status,
                                      static_cast<cudaStream_t>(stream));
}

// Projection kernel, then attention kernel, q / k / v through the caller's workspaces.
static int prefill_two_kernels(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                               void* q_ws, void* k_ws, void* v_ws, void* out, int B, int T, int window, float scale,
                               int value_dtype, int* status, void* stream) {
  int rc = fm_qkv_rope_bf16(x, w_qkv, cos, sin, cos_bstride, q_ws, k_ws, v_ws, B, T, value_dtype, status, stream);
  if (rc != 0) return rc;
  return fm_band_attn_prefill_bf16(q_ws, k_ws, v_ws, out, B, T, window, scale, value_dtype & 1, status, stream);
}

int fm_attention_prefill_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                              long long cos_bstride, void* q_ws, void* k_ws, void* v_ws, void* out, int B, int T,
                              int window, float scale, int value_dtype, int* status, void* stream) {
  // Whole clips of 129 .. 256 frames take the one-kernel form (projection + RoPE + attention, q / k / v never in
  // memory; the workspaces are not touched and may be null); every other length the projection kernel followed by
  // the attention kernel that fits it.
  if (T > 128 && T <= 256 && B > 0)
    return fm_attention_fused_bf16(x, w_qkv, cos, sin, cos_bstride, out, B, T, window, scale, value_dtype, status, stream);
  if (B > 0 && T > 0 && (q_ws == nullptr || k_ws == nullptr || v_ws == nullptr)) return -1;   // this form needs them
  return prefill_two_kernels(x, w_qkv, cos, sin, cos_bstride, q_ws, k_ws, v_ws, out, B, T, window, scale, value_dtype,
                             status, stream);
}

int fm_band_attn_chunk_bf16(const void* q, const void* k, const void* v, void* out, int B, int Tq, int Tk, int window,
                            float scale, int value_dtype, int* status, void* stream) {
  if (value_dtype != 0 && value_dtype != 1) return -1;
  return fm::launch_band_attn_chunk(q, k, v, out, B, Tq, Tk, window, scale, value_dtype, status,
                                    static_cast<cudaStream_t>(stream));
}

int fm_attention_fused_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                            void* out, int B, int T, int window, float scale, int value_dtype, int* status,
                            void* stream) {
  if (B < 0 || T < 0 || value_dtype < 0 || value_dtype > 3) return -1;
  if (B == 0 || T == 0) return 0;
  if (T <= 128 || T > 256) return -6;      // only whole clips of two 128-frame tiles
  return fm::launch_attn_fused_clip(x, w_qkv, cos, sin, cos_bstride, out, B, T, window, scale, value_dtype, status,
                                    static_cast<cudaStream_t>(stream));
}

int fm_attention_chunk_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                            void* q_ws, void* k_ws, void* v_ws, void* k_lin, void* v_lin, void* ring_k, void* ring_v,
                            void* out, int S, int T, int past, int ring_slots, int window, float scale, int value_dtype,
                            int* status, void* stream) {
  if (S < 0 || T < 0 || past < 0 || window <= 0 || ring_slots < window || value_dtype < 0 || value_dtype > 3) return -1;
  if (ring_k == nullptr || ring_v == nullptr) return -1;
  if (S == 0 || T == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = fm_qkv_rope_bf16(x, w_qkv, cos, sin, cos_bstride, q_ws, k_ws, v_ws, S, T, value_dtype, status, stream);
  if (rc != 0) return rc;
  const int delta = past < window - 1 ? past : window - 1;     // cached rows this call can still see
  if (delta == 0) {
    rc = fm::launch_band_attn_prefill(q_ws, k_ws, v_ws, out, S, T, window, scale, value_dtype & 1, status, st);
  } else {
    if (k_lin == nullptr || v_lin == nullptr) return -1;
    rc = fm::launch_ring_linearize(ring_k, ring_v, k_ws, v_ws, k_lin, v_lin, S, T, delta, past, ring_slots, st);
    if (rc != 0) return rc;
    rc = fm::launch_band_attn_chunk(q_ws, k_lin, v_lin, out, S, T, delta + T, window, scale, value_dtype & 1, status, st);
  }
  if (rc != 0) return rc;
  return fm::launch_ring_append(k_ws, v_ws, ring_k, ring_v, S, T, past, ring_slots, st);
}

int fm_out_proj_f16(const void* attn, const void* w_o, const float* layer_scale, const void* residual, void* y,
                    long long frames, int value_dtype, int* status, void* stream) {
  if (frames < 0 || frames > 0x7fffffffLL || value_dtype < 0 || value_dtype > 3) return -1;
  return fm::launch_out_proj_gemm(attn, w_o, y, layer_scale, residual, static_cast<int>(frames), value_dtype,
                                  status, static_cast<cudaStream_t>(stream));
}

int fm_linear_f16(const void* a, const void* w, const float* scale, const void* residual, void* y, long long rows,
                  int n_out, int k_in, int in_dtype, int out_dtype, int activation, int* status, void* stream) {
  if (rows < 0 || rows > 0x7fffffffLL || activation < 0 || activation > 1) return -1;
  return fm::launch_linear_gemm(a, w, y, scale, residual, static_cast<int>(rows), n_out, k_in, in_dtype, out_dtype,
                                activation, status, static_cast<cudaStream_t>(stream));
}

int fm_layernorm_f16(const void* x, int x_dtype, const float* weight, const float* bias, float eps, void* y,
                     int y_dtype, long long rows, void* stream) {
  return fm::launch_layernorm512(x, x_dtype, weight, bias, eps, y, y_dtype, rows, static_cast<cudaStream_t>(stream));
}

int fm_rvq_select_f32(const void* scores, int scores_dtype, const float* e_sq, const float* codebook, float* residual,
                      void* residual16, long long* codes, int* n_candidates, long long rows, int n_codes, float e_max,
                      float tau_rel, int* status, void* stream) {
  if (scores_dtype != 1 && scores_dtype != 2) return -1;
  return fm::launch_rvq_select(scores, scores_dtype == 1, e_sq, codebook, residual, residual16, codes, n_candidates, rows, n_codes, e_max,
                               tau_rel, status, static_cast<cudaStream_t>(stream));
}

int fm_conv_rows_split(const float* x, void* hi, void* lo, int B, int T, int C, int kernel, int stride, void* stream) {
  return fm::launch_conv_rows_split(x, hi, lo, B, T, C, kernel, stride, static_cast<cudaStream_t>(stream));
}

int fm_upsample2_f32(const float* x, const float* w, float* y, int B, int T, int C, void* stream) {
  return fm::launch_upsample2_depthwise(x, w, y, B, T, C, static_cast<cudaStream_t>(stream));
}

int fm_split_half(const float* x, void* hi, void* lo, long long n, void* stream) {
  return fm::launch_split_half(x, hi, lo, n, static_cast<cudaStream_t>(stream));
}

int fm_rvq_candidates_f16(const void* residual16, const void* codebook16, const float* e_sq, const float* tau,
                          void* records, long long rows, int n_codes, int* status, void* stream) {
  if (rows < 0 || rows > 0x7fffffffLL) return -1;
  return fm::launch_linear_gemm(residual16, codebook16, records, e_sq, tau, static_cast<int>(rows), n_codes, 256, 1, 3, 0,
                                status, static_cast<cudaStream_t>(stream));
}

int fm_rvq_select_rec_f32(const void* records, const float* codebook, float* residual, void* residual16, long long* codes,
                          int* n_candidates, float* tau, long long rows, int n_codes, float e_max_next, float tau_rel,
                          int* status, void* stream) {
  return fm::launch_rvq_select_rec(records, codebook, residual, residual16, codes, n_candidates, tau, rows, n_codes,
                                   e_max_next, tau_rel, status, static_cast<cudaStream_t>(stream));
}

int fm_rvq_prepare_f32(const float* x, void* residual16, float* tau, long long rows, float e_max, float tau_rel,
                       void* stream) {
  return fm::launch_rvq_prepare(x, residual16, tau, rows, e_max, tau_rel, static_cast<cudaStream_t>(stream));
}

int fm_rvq_to_half(const float* x, void* y, long long rows, void* stream) {
  return fm::launch_rvq_to_half(x, y, rows, static_cast<cudaStream_t>(stream));
}

int fm_rvq_decode_f32(const long long* codes, const float* codebooks, float* out, long long rows, int n_layers,
                      int n_codes, int* bad_code, void* stream) {
  return fm::launch_rvq_decode(codes, codebooks, out, rows, n_layers, n_codes, bad_code, static_cast<cudaStream_t>(stream));
}

int fm_ring_attn_decode_bf16(const void* q, const void* ring_k, const void* ring_v, float* out,
                             const int* stream_pos, int pos_base, int S, int ring_slots, float scale,
                             int value_dtype, int* status, void* stream) {
  if (value_dtype != 0 && value_dtype != 1) return -1;
  return fm::launch_ring_decode_attn(q, ring_k, ring_v, out, stream_pos, pos_base, S, ring_slots, scale,
                                     value_dtype, status, static_cast<cudaStream_t>(stream));
}

int fm_decode_step_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                        const int* stream_pos, int pos_base, void* q_ws, void* ring_k, void* ring_v, float* out,
                        int S, int ring_slots, float scale, int value_dtype, int* status, void* stream) {
  if (S < 0 || value_dtype < 0 || value_dtype > 3 || ring_slots <= 0 || ring_slots > 256 || pos_base < 0) return -1;
  if (ring_k == nullptr || ring_v == nullptr || q_ws == nullptr) return -1;
  QkvEpilogueArgs ep = {};
  ep.q = static_cast<uint16_t*>(q_ws);
  ep.ring_k = static_cast<uint16_t*>(ring_k);
  ep.ring_v = static_cast<uint16_t*>(ring_v);
  ep.cos = cos;
  ep.sin = sin;
  ep.cos_bstride = cos_bstride;
  ep.clip_pos = stream_pos;
  ep.pos_base = pos_base;
  ep.T = 1;
  ep.ring_slots = ring_slots;
  int rc = fm::launch_qkv_rope_gemm(x, w_qkv, ep, S, value_dtype, status, static_cast<cudaStream_t>(stream));
  if (rc != 0) return rc;
  return fm::launch_ring_decode_attn(q_ws, ring_k, ring_v, out, stream_pos, pos_base, S, ring_slots, scale,
                                     value_dtype & 1, status, static_cast<cudaStream_t>(stream));
}

int fm_band_attn_fp32_verify(const float* q, const float* k, const float* v, float* out, int B, int H, int D, int Tq,
                             int Tk, int q_off, int k_off, int window, float scale, const long long* strides,
                             void* stream) {
  if (strides == nullptr) return -1;
  return fm::launch_band_attn_fp32(q, k, v, out, B, H, D, Tq, Tk, q_off, k_off, window, scale, strides,
                                   static_cast<cudaStream_t>(stream));
}

int fm_linear_fp32_verify(const float* x, const float* w, float* y, int M, int N, int K, void* stream) {
  return fm::launch_linear_fp32(x, w, y, M, N, K, static_cast<cudaStream_t>(stream));
}

int fm_rope_fp32_verify(float* t, const float* cos, const float* sin, int B, int T, int H, int D,
                        long long cos_bstride, void* stream) {
  return fm::launch_rope_fp32(t, cos, sin, B, T, H, D, cos_bstride, static_cast<cudaStream_t>(stream));
}

// ---- entry point that allocates nothing -----------------------------------------------------------
// Workspace for fm_attention_prefill_static_bf16: rotated q, k and v of up to FM_STATIC_MAX_FRAMES frames
// (3 x 8192 x 512 x 2 B = 24 MiB).  It is part of the loaded module image, so every GPU that loads the
// library holds it until the process exits.
static __device__ __align__(256) unsigned short g_static_qkv[3ull * FM_STATIC_MAX_FRAMES * 512];

// Device address of g_static_qkv on the current device.  In host code the array's name is only a handle
// for the runtime, not something a kernel can dereference, so the address is asked for once per device.
static int static_workspace(unsigned short** out) {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static unsigned short* ptrs[kMaxDev];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDev) return -1;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_qkv);
    if (e != cudaSuccess) return static_cast<int>(e);
    ptrs[dev] = static_cast<unsigned short*>(p);
  }
  *out = ptrs[dev];
  return 0;
}

int fm_attention_prefill_static_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                                     long long cos_bstride, void* out, int B, int T, int window, float scale,
                                     int value_dtype, int* status, void* stream) {
  if (B < 0 || T < 0) return -1;
  const long long frames = static_cast<long long>(B) * T;
  if (frames > FM_STATIC_MAX_FRAMES) return -5;     // larger than the built-in workspace
  if (frames == 0) return 0;
  unsigned short* ws = nullptr;
  const int rc = static_workspace(&ws);
  if (rc != 0) return rc;
  unsigned short* q_ws = ws;
  unsigned short* k_ws = ws + frames * 512;
  unsigned short* v_ws = ws + 2 * frames * 512;
  // always the two-kernel path: this entry point exists to supply the q / k / v workspace
  return prefill_two_kernels(x, w_qkv, cos, sin, cos_bstride, q_ws, k_ws, v_ws, out, B, T, window, scale, value_dtype,
                             status, stream);
}

int fm_selftest_wait_timeout(int* status, int limit_us, int* observed, void* stream) {
  return fm::launch_wait_timeout_selftest(status, limit_us, observed, static_cast<cudaStream_t>(stream));
}

int fm_read_status(const int* status, void* stream) {
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  if (status == nullptr) return 0;
  int host = 0;
  e = cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  return host;
}

}  // extern "C"
