// Kernels on the float32 residual stream for blocks that do more than add a sublayer's output:
//
//   embed_pair        x = table[token] * scale + pair_table[row], row = (previous token * a + token * b)
//                     mod buckets, row `buckets` for a sequence's first token; the previous token of a
//                     portion's first row comes from the request's state slot
//   last_token_update the state slot's token after a step: the last token of each sequence
//   norm_conv         h = rmsnorm(x) w, out = h + conv(h): a causal convolution over time on every
//                     channel, conv(h)_t = sum_j c[:, j] h_(t - taps + 1 + j); rows before the step's
//                     first come from the request's state slot, zeros before position 0; h is kept
//                     for the rows that the state holds after the step
//   scaled_add        x += s * d per channel (or nothing added), optionally also x in the activation type
//   token_gate        g = gelu_tanh(t) * e[token], e a slice of a per-token table
//   normed_add_mix    x += m * y / rms(y) * w (y optional), keep the row as entry `index` of the row's
//                     history, then x = sum_j a[j] * history[j], j = 0 .. index
//   copy_history      history entry 0 of every row = x
//
// Everything is float32 in both precisions; only tables that are loaded and activations that are
// stored change type. Sums run in an order that the sizes alone fix.
#include "bw_act.cuh"

#include <math.h>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxTaps = 16;

__global__ void __launch_bounds__(128)
embed_pair_kernel(const act_t* __restrict__ table, const act_t* __restrict__ pair_table, const int* __restrict__ tokens,
                  const int* __restrict__ pos, const int* __restrict__ row_seq, const int* __restrict__ seq_row0,
                  const int* __restrict__ seq_slot, const int* __restrict__ last_token, float* __restrict__ out, int width,
                  float scale, int buckets, int mul_prev, int mul_cur) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int tok = tokens[r];
  const act_t* src = table + static_cast<size_t>(tok) * width;
  float* dst = out + static_cast<size_t>(r) * width;
  if (!pair_table) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = __fmul_rn(bw::to_f(src[i]), scale);
    return;
  }
  const int seq = row_seq[r];
  long long row = buckets;
  if (pos[r] > 0) {
    const int prev = r > seq_row0[seq] ? tokens[r - 1] : last_token[seq_slot[seq]];
    row = (static_cast<long long>(prev) * mul_prev + static_cast<long long>(tok) * mul_cur) % buckets;
  }
  const act_t* pair = pair_table + static_cast<size_t>(row) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = __fadd_rn(__fmul_rn(bw::to_f(src[i]), scale), bw::to_f(pair[i]));
}

__global__ void last_token_update_kernel(const int* __restrict__ tokens, const int* __restrict__ tile_seq,
                                         const int* __restrict__ tile_row0, const int* __restrict__ tile_rows, int tiles,
                                         const int* __restrict__ seq_slot, int* last_token) {
  bw::pdl_enter();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tiles) return;
  last_token[seq_slot[tile_seq[t]]] = tokens[tile_row0[t] + tile_rows[t] - 1];
}

// A block takes `rows_per_block` consecutive rows of the step (at most kConvRows) and the channels [c0, c0 +
// chans) of them. Its warps first form 1 / rms of those rows and of the taps - 1 rows before them that belong
// to the first row's sequence, a row per warp at a time (the same arithmetic whichever block forms a row and
// however the step is cut, so a row's normed values are the same bits as the row itself and as the rows after
// it see them); then every thread walks its channels down the block's rows, with the normed values of the
// taps - 1 rows before in registers. Rows before the step's first of a sequence come from the request's state
// slot. `normed` is written only where `conv_state_update` reads it: the last taps - 1 rows of a sequence's
// portion.
constexpr int kConvRows = 8;

int sm_count() {
  static int sms = 0;
  if (sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

template <int kTaps /* 0: any number up to kMaxTaps, rows before read again */>
__global__ void __launch_bounds__(kThreads)
norm_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, const float* __restrict__ taps_t,
                 int taps_any, const float* __restrict__ state, int state_cols, int state_col0, const int* __restrict__ pos,
                 const int* __restrict__ row_seq, const int* __restrict__ seq_row0, const int* __restrict__ seq_slot,
                 act_t* __restrict__ out, float* __restrict__ normed, int normed_cols, int normed_col0, int n, int width,
                 int rows_per_block, int chans) {
  bw::pdl_enter();
  const int taps = kTaps ? kTaps : taps_any;
  __shared__ float inv_of[kConvRows + kMaxTaps];  // entry j: row r0 - (taps - 1) + j
  __shared__ int row_pos[kConvRows], row_first[kConvRows], row_slot[kConvRows], row_keep[kConvRows];
  const int r0 = blockIdx.x * rows_per_block;
  const int rows = min(rows_per_block, n - r0);
  const int first = r0 - (taps - 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq0 = row_seq[r0];
  for (int j = warp; j < rows + taps - 1; j += kThreads / 32) {
    const int rr = first + j;
    if (rr < 0 || (rr < r0 && row_seq[rr] != seq0)) continue;  // (uniform over the warp)
    const float* xr = x + static_cast<size_t>(rr) * width;
    float ss = 0.0f;
#pragma unroll 8
    for (int i = lane; i < width; i += 32) ss = __fmaf_rn(xr[i], xr[i], ss);
    ss = bw::warp_sum(ss);
    if (lane == 0) inv_of[j] = bw::rms_scale(ss, width, eps);
  }
  if (threadIdx.x < rows) {
    const int r = r0 + threadIdx.x;
    const int seq = row_seq[r];
    const int ahead = r + taps - 1;  // the row's place in the state after the step: among its sequence's last taps - 1
    row_pos[threadIdx.x] = pos[r];
    row_first[threadIdx.x] = seq_row0[seq];
    row_slot[threadIdx.x] = seq_slot[seq];
    row_keep[threadIdx.x] = taps > 1 && (ahead >= n || row_seq[ahead] != seq);
  }
  __syncthreads();
  const int c0 = blockIdx.y * chans;
  const int c1 = min(width, c0 + chans);
  for (int i = c0 + threadIdx.x; i < c1; i += kThreads) {
    const float wi = w[i];
    if constexpr (kTaps != 0) {
      float c[kTaps], h[kTaps];  // h[t]: the normed value of row r - (kTaps - 1) + t, where the step has that row
#pragma unroll
      for (int t = 0; t < kTaps; ++t) c[t] = taps_t[static_cast<size_t>(t) * width + i];
#pragma unroll
      for (int t = 0; t + 1 < kTaps; ++t) {
        const int rr = first + t;
        h[t + 1] = rr >= row_first[0] ? bw::rms_apply(x[static_cast<size_t>(rr) * width + i], inv_of[t], wi) : 0.0f;
      }
      for (int j = 0; j < rows; ++j) {
        const int r = r0 + j;
        const int p = row_pos[j], row0 = row_first[j];
#pragma unroll
        for (int t = 0; t + 1 < kTaps; ++t) h[t] = h[t + 1];
        h[kTaps - 1] = bw::rms_apply(x[static_cast<size_t>(r) * width + i], inv_of[j + kTaps - 1], wi);
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < kTaps; ++t) {  // taps ascending
          const int back = kTaps - 1 - t;
          if (p - back < 0) continue;
          float hv = h[t];
          if (r - back < row0)
            hv = state[(static_cast<size_t>(row_slot[j]) * (kTaps - 1) + (kTaps - 1 - (row0 - (r - back)))) * state_cols +
                       state_col0 + i];
          acc = __fmaf_rn(c[t], hv, acc);
        }
        if (row_keep[j]) normed[static_cast<size_t>(r) * normed_cols + normed_col0 + i] = h[kTaps - 1];
        out[static_cast<size_t>(r) * width + i] = bw::from_f<act_t>(__fadd_rn(h[kTaps - 1], acc));
      }
    } else {
      for (int j = 0; j < rows; ++j) {
        const int r = r0 + j;
        const int p = row_pos[j], row0 = row_first[j];
        const float own = bw::rms_apply(x[static_cast<size_t>(r) * width + i], inv_of[j + taps - 1], wi);
        float acc = 0.0f;
        for (int t = 0; t < taps; ++t) {  // taps ascending
          const int back = taps - 1 - t;
          if (p - back < 0) continue;
          const int rr = r - back;
          float hv;
          if (back == 0)
            hv = own;
          else if (rr >= row0)
            hv = bw::rms_apply(x[static_cast<size_t>(rr) * width + i], inv_of[j + t], wi);
          else
            hv = state[(static_cast<size_t>(row_slot[j]) * (taps - 1) + (taps - 1 - (row0 - rr))) * state_cols + state_col0 + i];
          acc = __fmaf_rn(taps_t[static_cast<size_t>(t) * width + i], hv, acc);
        }
        if (row_keep[j]) normed[static_cast<size_t>(r) * normed_cols + normed_col0 + i] = own;
        out[static_cast<size_t>(r) * width + i] = bw::from_f<act_t>(__fadd_rn(own, acc));
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads)
scaled_add_kernel(float* x, const float* __restrict__ s, const float* __restrict__ d, act_t* __restrict__ rounded,
                  int width) {
  bw::pdl_enter();
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float v = x[base + i];
    if (s) {
      v = __fmaf_rn(s[i], d[base + i], v);
      x[base + i] = v;
    }
    if (rounded) rounded[base + i] = bw::from_f<act_t>(v);
  }
}

__device__ __forceinline__ float gelu_tanh(float z) {
  const float inner = __fmul_rn(0.7978845608028654f, __fmaf_rn(__fmul_rn(0.044715f, z), __fmul_rn(z, z), z));
  return __fmul_rn(__fmul_rn(0.5f, z), __fadd_rn(1.0f, tanhf(inner)));
}

__global__ void token_gate_kernel(const float* __restrict__ t, const act_t* __restrict__ table, int table_cols, int col0,
                                  const int* __restrict__ tokens, act_t* __restrict__ out, int n, int dim) {
  bw::pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * dim) return;
  const int r = idx / dim, c = idx - r * dim;
  const float e = bw::to_f(table[static_cast<size_t>(tokens[r]) * table_cols + col0 + c]);
  out[idx] = bw::from_f<act_t>(__fmul_rn(gelu_tanh(t[idx]), e));
}

__global__ void __launch_bounds__(kThreads)
normed_add_mix_kernel(float* x, const float* __restrict__ y, const float* __restrict__ w, float eps, float mult,
                      float* history, int entries, int index, const float* __restrict__ mix, int width) {
  bw::pdl_enter();
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float inv = 0.0f;
  if (y) {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += kThreads) ss = __fmaf_rn(y[base + i], y[base + i], ss);
    inv = bw::rms_scale(bw::block_sum(ss, red), width, eps);
  }
  float* hist = history ? history + static_cast<size_t>(blockIdx.x) * entries * width : nullptr;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float v = x[base + i];
    if (y) v = __fmaf_rn(mult, bw::rms_apply(y[base + i], inv, w[i]), v);
    if (hist) {
      hist[static_cast<size_t>(index) * width + i] = v;
      float acc = 0.0f;
      for (int j = 0; j < index; ++j) acc = __fmaf_rn(mix[j], hist[static_cast<size_t>(j) * width + i], acc);
      v = __fmaf_rn(mix[index], v, acc);
    }
    x[base + i] = v;
  }
}

__global__ void __launch_bounds__(kThreads)
copy_history_kernel(const float* __restrict__ x, float* __restrict__ history, int entries, int width) {
  bw::pdl_enter();
  const float* src = x + static_cast<size_t>(blockIdx.x) * width;
  float* dst = history + static_cast<size_t>(blockIdx.x) * entries * width;
  for (int i = threadIdx.x; i < width; i += kThreads) dst[i] = src[i];
}

}  // namespace

BW_API int BW_FN(embed_pair)(const void* table, const void* pair_table, const int* tokens, const int* pos,
                             const int* row_seq, const int* seq_row0, const int* seq_slot, const int* last_token, float* out,
                             int n, int width, float scale, int buckets, int mul_prev, int mul_cur, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (pair_table && (buckets <= 0 || !last_token)) {
    bw::set_error("embed_pair: %d buckets, or no state for the previous token", buckets);
    return -1;
  }
  bw::launch_pdl(embed_pair_kernel, dim3(n), dim3(128), 0, stream, static_cast<const act_t*>(table),
                 static_cast<const act_t*>(pair_table), tokens, pos, row_seq, seq_row0, seq_slot, last_token, out, width, scale,
                 buckets, mul_prev, mul_cur);
  return bw::launch_status();
}

BW_API int BW_FN(last_token_update)(const int* tokens, const int* tile_seq, const int* tile_row0, const int* tile_rows,
                                    int tiles, const int* seq_slot, int* last_token, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  bw::launch_pdl(last_token_update_kernel, dim3((tiles + 63) / 64), dim3(64), 0, stream, tokens, tile_seq, tile_row0,
                 tile_rows, tiles, seq_slot, last_token);
  return bw::launch_status();
}

BW_API int BW_FN(norm_conv)(const float* x, const float* w, float eps, const float* taps_t, int taps, const float* state,
                            int state_cols, int state_col0, const int* pos, const int* row_seq, const int* seq_row0,
                            const int* seq_slot, void* out, float* normed, int normed_cols, int normed_col0, int n,
                            int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps || (taps > 1 && !state)) {
    bw::set_error("norm_conv: %d taps (1 .. %d, with the requests' state from 2 on)", taps, kMaxTaps);
    return -1;
  }
  // rows per block and channels per block: enough blocks to fill the device where the step has the work for it
  const int rows_per_block = n >= kConvRows * 2 * sm_count() ? kConvRows : max(1, min(kConvRows, n / sm_count()));
  const int groups = (n + rows_per_block - 1) / rows_per_block;
  int slices = max(1, min((width + kThreads - 1) / kThreads, (2 * sm_count() + groups - 1) / groups));
  const int chans = ((width + slices - 1) / slices + 31) / 32 * 32;
  slices = (width + chans - 1) / chans;
  auto go = [&](auto kernel) {
    bw::launch_pdl(kernel, dim3(groups, slices), dim3(kThreads), 0, stream, x, w, eps, taps_t, taps, state, state_cols,
                   state_col0, pos, row_seq, seq_row0, seq_slot, static_cast<act_t*>(out), normed, normed_cols, normed_col0, n,
                   width, rows_per_block, chans);
  };
  switch (taps) {
    case 1: go(norm_conv_kernel<1>); break;
    case 2: go(norm_conv_kernel<2>); break;
    case 3: go(norm_conv_kernel<3>); break;
    case 4: go(norm_conv_kernel<4>); break;
    default: go(norm_conv_kernel<0>); break;
  }
  return bw::launch_status();
}

BW_API int BW_FN(scaled_add)(float* x, const float* s, const float* d, void* rounded, int n, int width,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  bw::launch_pdl(scaled_add_kernel, dim3(n), dim3(kThreads), 0, stream, x, s, d, static_cast<act_t*>(rounded), width);
  return bw::launch_status();
}

BW_API int BW_FN(token_gate)(const float* t, const void* table, int table_cols, int col0, const int* tokens, void* out,
                             int n, int dim, cudaStream_t stream) {
  if (n <= 0 || dim <= 0) return 0;
  bw::launch_pdl(token_gate_kernel, dim3((n * dim + 255) / 256), dim3(256), 0, stream, t,
                 static_cast<const act_t*>(table), table_cols, col0, tokens, static_cast<act_t*>(out), n, dim);
  return bw::launch_status();
}

BW_API int BW_FN(normed_add_mix)(float* x, const float* y, const float* w, float eps, float mult, float* history,
                                 int entries, int index, const float* mix, int n, int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (history && (index < 0 || index >= entries || !mix)) {
    bw::set_error("normed_add_mix: entry %d of a history of %d", index, entries);
    return -1;
  }
  bw::launch_pdl(normed_add_mix_kernel, dim3(n), dim3(kThreads), 0, stream, x, y, w, eps, mult, history, entries, index,
                 mix, width);
  return bw::launch_status();
}

BW_API int BW_FN(copy_history)(const float* x, float* history, int entries, int n, int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  bw::launch_pdl(copy_history_kernel, dim3(n), dim3(kThreads), 0, stream, x, history, entries, width);
  return bw::launch_status();
}
