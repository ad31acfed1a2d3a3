// Layer norm with a weight and no bias, and the row-wise helpers of blocks whose mixer and
// feed-forward read the same input: y = (x - mean) / sqrt(var + eps) * w, var the mean of the
// squared deviations (two passes over a row held in shared memory). Statistics and the stream
// are float32 in both precisions. One block per row; a row's sums are formed in an order that
// depends on the width only.
#include "bw_act.cuh"

namespace {

constexpr int kThreads = 256;

// Up to two outputs with weights of their own share one pass over the row (the two norms of a
// parallel block see the same x, hence the same mean and variance). An output may be the input
// itself (the norm after the embedding works in place on the stream).
template <typename OutT>
__global__ void __launch_bounds__(kThreads)
layernorm_kernel(const float* x, const float* __restrict__ w1, const float* __restrict__ w2, OutT* y1, OutT* y2,
                 const int* __restrict__ rows, int width, float eps) {
  bw::pdl_enter();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + static_cast<size_t>(src) * width;
  float s = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float v = xr[i];
    row[i] = v;
    s = __fadd_rn(s, v);
  }
  const float mean = __fdiv_rn(bw::block_sum(s, red), static_cast<float>(width));
  float q = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float d = __fsub_rn(row[i], mean);
    q = __fmaf_rn(d, d, q);
  }
  const float var = __fdiv_rn(bw::block_sum(q, red), static_cast<float>(width));
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
  OutT* o1 = y1 + static_cast<size_t>(r) * width;
  OutT* o2 = y2 ? y2 + static_cast<size_t>(r) * width : nullptr;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float n = __fmul_rn(__fsub_rn(row[i], mean), inv);
    o1[i] = bw::from_f<OutT>(__fmul_rn(n, w1[i]));
    if (o2) o2[i] = bw::from_f<OutT>(__fmul_rn(n, w2[i]));
  }
}

// The layer norm that follows a sublayer in blocks with a norm on both sides of each sublayer:
// x += (d - mean(d)) / sqrt(var(d) + eps) * w, with d the sublayer's output (float32) and x the
// float32 stream; a constant factor on what is added is folded into w by the caller. Where the
// next sublayer's layer norm follows at once, the same block forms it from the row it has just
// summed: xn = (x - mean(x)) / sqrt(var(x) + eps') * w', one kernel instead of two.
__global__ void __launch_bounds__(kThreads)
layernorm_residual_kernel(const float* __restrict__ d, const float* __restrict__ w, float* x, int width, float eps,
                          const float* __restrict__ w_next, float eps_next, act_t* xn) {
  bw::pdl_enter();
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  const float fw = static_cast<float>(width);
  float s = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float v = d[base + i];
    row[i] = v;
    s = __fadd_rn(s, v);
  }
  const float mean = __fdiv_rn(bw::block_sum(s, red), fw);
  float q = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float c = __fsub_rn(row[i], mean);
    q = __fmaf_rn(c, c, q);
  }
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(bw::block_sum(q, red), fw), eps)));
  float s2 = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float v = __fadd_rn(x[base + i], __fmul_rn(__fmul_rn(__fsub_rn(row[i], mean), inv), w[i]));
    x[base + i] = v;
    row[i] = v;  // (each thread reads back only what it wrote)
    s2 = __fadd_rn(s2, v);
  }
  if (!xn) return;
  const float mean2 = __fdiv_rn(bw::block_sum(s2, red), fw);
  float q2 = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float c = __fsub_rn(row[i], mean2);
    q2 = __fmaf_rn(c, c, q2);
  }
  const float inv2 = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(bw::block_sum(q2, red), fw), eps_next)));
  for (int i = threadIdx.x; i < width; i += kThreads)
    xn[base + i] = bw::from_f<act_t>(__fmul_rn(__fmul_rn(__fsub_rn(row[i], mean2), inv2), w_next[i]));
}

// x += d, element by element (the residual sum of a block whose parts wrote into d).
__global__ void add_rows_kernel(float* x, const float* __restrict__ d, size_t count) {
  bw::pdl_enter();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) x[i] = __fadd_rn(x[i], d[i]);
}

}  // namespace

// out_is_f32: y1 / y2 are float32 (else the precision's activation type). y2 and w2 may be null.
BW_API int BW_FN(layernorm)(const float* x, const float* w1, const float* w2, void* y1, void* y2, int out_is_f32,
                            const int* rows, int n, int width, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0 || width > 48 * 1024 / 4) {
    bw::set_error("layernorm: width %d (1 .. 12288)", width);
    return -1;
  }
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  if (out_is_f32)
    bw::launch_pdl(layernorm_kernel<float>, dim3(n), dim3(kThreads), smem, stream, x, w1, w2, static_cast<float*>(y1),
                   static_cast<float*>(y2), rows, width, eps);
  else
    bw::launch_pdl(layernorm_kernel<act_t>, dim3(n), dim3(kThreads), smem, stream, x, w1, w2, static_cast<act_t*>(y1),
                   static_cast<act_t*>(y2), rows, width, eps);
  return bw::launch_status();
}

// w_next, xn: the layer norm of the summed row into xn (activation type) as well; both null for none.
BW_API int BW_FN(layernorm_residual)(const float* d, const float* w, float* x, int n, int width, float eps,
                                     const float* w_next, float eps_next, void* xn, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0 || width > 48 * 1024 / 4) {
    bw::set_error("layernorm_residual: width %d (1 .. 12288)", width);
    return -1;
  }
  bw::launch_pdl(layernorm_residual_kernel, dim3(n), dim3(kThreads), static_cast<size_t>(width) * sizeof(float), stream,
                 d, w, x, width, eps, w_next, eps_next, static_cast<act_t*>(w_next ? xn : nullptr));
  return bw::launch_status();
}

BW_API int BW_FN(add_rows)(float* x, const float* d, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  const int threads = 256;
  bw::launch_pdl(add_rows_kernel, dim3(static_cast<unsigned>((count + threads - 1) / threads)), dim3(threads), 0, stream,
                 x, d, static_cast<size_t>(count));
  return bw::launch_status();
}
