// Small element-wise steps of gated designs, float32 arithmetic in both precisions:
//   sigmoid_gate   the output gate of a mixer: the heads' outputs times sigmoid(g), with one gate
//                  number per entry or one per group of neighbouring entries (a head)
//   glu_gelu       the gated feed-forward's inner step with the tanh form of GELU:
//                  h = gelu_tanh(gate) * up for rows laid out [gate | up]
//   softcap_rows   z <- cap * tanh(z / cap) on float32 rows (the logits' cap)
#include "bw_act.cuh"

#include <math.h>
#include <stdint.h>

namespace {

#if !BW_ACT_BF16
constexpr float kGeluCubic = 0.044715f;
constexpr float kSqrt2OverPi = 0.7978845608028654f;
#endif

__device__ __forceinline__ float sigmoid_f(float z) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z))); }

#if !BW_ACT_BF16
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float gelu_tanh_f(float z) {
  const float inner = __fmul_rn(kSqrt2OverPi, __fmaf_rn(__fmul_rn(kGeluCubic, __fmul_rn(z, z)), z, z));
  return __fmul_rn(__fmul_rn(0.5f, z), __fadd_rn(1.0f, tanhf(inner)));
}
#endif

// v[r][c] *= sigmoid(g[r][c / group]); g is float32 with a row stride of its own.
__global__ void sigmoid_gate_kernel(act_t* v, int cols, const float* __restrict__ g, int g_stride, int group, size_t count) {
  bw::pdl_enter();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const size_t r = i / cols;
  const int c = static_cast<int>(i - r * cols);
  v[i] = bw::from_f<act_t>(__fmul_rn(bw::to_f(v[i]), sigmoid_f(g[r * g_stride + c / group])));
}

// The same for rows whose length is a multiple of 8, with groups of one entry or of a multiple of 8: a thread takes
// 8 neighbouring entries (16 or 32 bytes at a time) of the row blockIdx.x.
__global__ void __launch_bounds__(256)
sigmoid_gate_vec_kernel(act_t* v, int cols, const float* __restrict__ g, int g_stride, int group) {
  bw::pdl_enter();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  const size_t r = blockIdx.x;
  act_t* at = v + r * cols + c;
  float s[8];
  if (group == 1) {
    const float4 a = *reinterpret_cast<const float4*>(g + r * g_stride + c), b = *reinterpret_cast<const float4*>(g + r * g_stride + c + 4);
    s[0] = a.x, s[1] = a.y, s[2] = a.z, s[3] = a.w, s[4] = b.x, s[5] = b.y, s[6] = b.z, s[7] = b.w;
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = sigmoid_f(s[e]);
  } else {
    const float one = sigmoid_f(g[r * g_stride + c / group]);
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = one;
  }
#if BW_ACT_BF16
  uint4 raw = *reinterpret_cast<const uint4*>(at);
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    h[e] = __floats2bfloat162_rn(__fmul_rn(f.x, s[2 * e]), __fmul_rn(f.y, s[2 * e + 1]));
  }
  *reinterpret_cast<uint4*>(at) = raw;
#else
  float4 a = *reinterpret_cast<const float4*>(at), b = *reinterpret_cast<const float4*>(at + 4);
  a.x = __fmul_rn(a.x, s[0]), a.y = __fmul_rn(a.y, s[1]), a.z = __fmul_rn(a.z, s[2]), a.w = __fmul_rn(a.w, s[3]);
  b.x = __fmul_rn(b.x, s[4]), b.y = __fmul_rn(b.y, s[5]), b.z = __fmul_rn(b.z, s[6]), b.w = __fmul_rn(b.w, s[7]);
  *reinterpret_cast<float4*>(at) = a, *reinterpret_cast<float4*>(at + 4) = b;
#endif
}

__global__ void glu_gelu_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inter, size_t count) {
  bw::pdl_enter();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const size_t r = i / inter;
  const int c = static_cast<int>(i - r * inter);
  const act_t* g = gate_up + r * 2 * inter + c;
#if BW_ACT_BF16
  // the serving precision's form, shared with the epilogue of the gate/up product: both give the same bits
  out[i] = bw::from_f<act_t>(bw::geglu_one(bw::to_f(g[0]), bw::to_f(g[inter])));
#else
  out[i] = bw::from_f<act_t>(__fmul_rn(gelu_tanh_f(bw::to_f(g[0])), bw::to_f(g[inter])));
#endif
}

__global__ void softcap_rows_kernel(float* z, float cap, size_t count) {
  bw::pdl_enter();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) z[i] = __fmul_rn(cap, tanhf(__fdiv_rn(z[i], cap)));
}

unsigned blocks_for(size_t count) { return static_cast<unsigned>((count + 255) / 256); }

}  // namespace

// v: [n, cols] in the activation type, gated in place; g: float32 rows of `g_stride` floats holding
// cols / group gate numbers each.
BW_API int BW_FN(sigmoid_gate)(void* v, int n, int cols, const float* g, int g_stride, int group, cudaStream_t stream) {
  if (n <= 0 || cols <= 0) return 0;
  if (group <= 0 || cols % group) {
    bw::set_error("sigmoid_gate: %d columns are not whole groups of %d", cols, group);
    return -1;
  }
  const bool aligned = reinterpret_cast<uintptr_t>(v) % 32 == 0 &&
                       (group > 1 || (reinterpret_cast<uintptr_t>(g) % 16 == 0 && g_stride % 4 == 0));
  if (cols % 8 == 0 && (group == 1 || group % 8 == 0) && aligned) {
    const int threads = cols / 8 >= 256 ? 256 : (cols / 8 + 31) / 32 * 32;
    bw::launch_pdl(sigmoid_gate_vec_kernel, dim3(n, (cols / 8 + threads - 1) / threads), dim3(threads), 0, stream, static_cast<act_t*>(v), cols, g,
                   g_stride, group);
    return bw::launch_status();
  }
  const size_t count = static_cast<size_t>(n) * cols;
  bw::launch_pdl(sigmoid_gate_kernel, dim3(blocks_for(count)), dim3(256), 0, stream, static_cast<act_t*>(v), cols, g,
                 g_stride, group, count);
  return bw::launch_status();
}

BW_API int BW_FN(glu_gelu)(const void* gate_up, void* out, int n, int inter, cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  const size_t count = static_cast<size_t>(n) * inter;
  bw::launch_pdl(glu_gelu_kernel, dim3(blocks_for(count)), dim3(256), 0, stream, static_cast<const act_t*>(gate_up),
                 static_cast<act_t*>(out), inter, count);
  return bw::launch_status();
}

BW_API int BW_FN(softcap_rows)(float* z, long long count, float cap, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.0f)) {
    bw::set_error("softcap_rows: the cap must be positive, got %g", static_cast<double>(cap));
    return -1;
  }
  bw::launch_pdl(softcap_rows_kernel, dim3(blocks_for(static_cast<size_t>(count))), dim3(256), 0, stream, z, cap,
                 static_cast<size_t>(count));
  return bw::launch_status();
}
