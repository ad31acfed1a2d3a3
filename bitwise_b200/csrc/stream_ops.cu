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
constexpr int kConvThreads = 512;  // one round of sums for eight rows and the rows before them

int sm_count() {
  static int sms = 0;
  if (sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// A lane's share of a row's sum of squares: the quads lane, lane + 32, ... of the row, one running sum per place
// in the quad, then the tail. The order is the same with 16-byte loads and without, so the bits do not depend on
// where the row lies.
__device__ __forceinline__ float lane_sumsq(const float* __restrict__ xr, int width, int lane, bool vec) {
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  const int quads = width >> 2;
  if (vec) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
#pragma unroll 8
    for (int q = lane; q < quads; q += 32) {
      const float4 v = x4[q];
      a0 = __fmaf_rn(v.x, v.x, a0);
      a1 = __fmaf_rn(v.y, v.y, a1);
      a2 = __fmaf_rn(v.z, v.z, a2);
      a3 = __fmaf_rn(v.w, v.w, a3);
    }
  } else {
    for (int q = lane; q < quads; q += 32) {
      const float* v = xr + 4 * q;
      a0 = __fmaf_rn(v[0], v[0], a0);
      a1 = __fmaf_rn(v[1], v[1], a1);
      a2 = __fmaf_rn(v[2], v[2], a2);
      a3 = __fmaf_rn(v[3], v[3], a3);
    }
  }
  for (int i = (quads << 2) + lane; i < width; i += 32) a0 = __fmaf_rn(xr[i], xr[i], a0);
  return __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
}

template <int kTaps /* 0: any number up to kMaxTaps, rows before read again */>
__global__ void __launch_bounds__(kConvThreads, 2)
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
  const bool vec = (width & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  // what the first threads look up about the block's rows is asked for before the sums, and what depends on the
  // answers between the two rounds of sums, so that no lookup is waited for alone
  const bool meta = threadIdx.x < rows;
  int m_pos = 0, m_seq = 0, m_ahead = -1;
  if (meta) {
    const int r = r0 + threadIdx.x;
    const int ahead = r + taps - 1;  // the row's place in the state after the step: among its sequence's last taps - 1
    m_pos = pos[r];
    m_seq = row_seq[r];
    if (ahead < n) m_ahead = row_seq[ahead];
  }
  const int seq0 = row_seq[r0];
  for (int j = warp; j < rows; j += kConvThreads / 32) {  // the block's own rows
    const float ss = bw::warp_sum(lane_sumsq(x + static_cast<size_t>(r0 + j) * width, width, lane, vec));
    if (lane == 0) inv_of[taps - 1 + j] = bw::rms_scale(ss, width, eps);
  }
  int m_first = 0, m_slot = 0;
  if (meta) {
    m_first = seq_row0[m_seq];
    m_slot = seq_slot[m_seq];
  }
  for (int t = warp; t < taps - 1; t += kConvThreads / 32) {  // the rows before them that the first row's sequence has
    const int rr = first + t;
    if (rr < 0 || row_seq[rr] != seq0) continue;  // (uniform over the warp)
    const float ss = bw::warp_sum(lane_sumsq(x + static_cast<size_t>(rr) * width, width, lane, vec));
    if (lane == 0) inv_of[t] = bw::rms_scale(ss, width, eps);
  }
  if (meta) {
    row_pos[threadIdx.x] = m_pos;
    row_first[threadIdx.x] = m_first;
    row_slot[threadIdx.x] = m_slot;
    // bit 0: the state keeps the row; bit 1: the step holds all taps - 1 rows before it
    row_keep[threadIdx.x] = (taps > 1 && m_ahead != m_seq ? 1 : 0) |
                            (m_pos >= taps - 1 && r0 + static_cast<int>(threadIdx.x) - (taps - 1) >= m_first ? 2 : 0);
  }
  __syncthreads();
  const int c0 = blockIdx.y * chans;
  const int c1 = min(width, c0 + chans);
  for (int i = c0 + threadIdx.x; i < c1; i += kConvThreads) {
    const float wi = w[i];
    if constexpr (kTaps != 0) {
      // the block's rows and the kTaps - 1 before them, loaded together: h[t] is the normed value of row first + t,
      // where the step has that row for the first row's sequence (the rows of a later sequence all lie in the block)
      float c[kTaps], h[kConvRows + kTaps - 1];
#pragma unroll
      for (int t = 0; t < kTaps; ++t) c[t] = taps_t[static_cast<size_t>(t) * width + i];
#pragma unroll
      for (int t = 0; t < kConvRows + kTaps - 1; ++t) {
        const int rr = first + t;
        const bool have = t < rows + kTaps - 1 && (t >= kTaps - 1 || rr >= row_first[0]);
        h[t] = have ? x[static_cast<size_t>(rr) * width + i] : 0.0f;
      }
#pragma unroll
      for (int t = 0; t < kConvRows + kTaps - 1; ++t) {
        const bool have = t < rows + kTaps - 1 && (t >= kTaps - 1 || first + t >= row_first[0]);
        if (have) h[t] = bw::rms_apply(h[t], inv_of[t], wi);
      }
#pragma unroll
      for (int j = 0; j < kConvRows; ++j) {
        if (j < rows) {
          const int r = r0 + j;
          const int flags = row_keep[j];
          float acc = 0.0f;
          if (flags & 2) {
#pragma unroll
            for (int t = 0; t < kTaps; ++t) acc = __fmaf_rn(c[t], h[j + t], acc);  // taps ascending
          } else {
            const int p = row_pos[j], row0 = row_first[j];
#pragma unroll
            for (int t = 0; t < kTaps; ++t) {
              const int back = kTaps - 1 - t;
              if (p - back < 0) continue;
              float hv = h[j + t];
              if (r - back < row0)
                hv = state[(static_cast<size_t>(row_slot[j]) * (kTaps - 1) + (kTaps - 1 - (row0 - (r - back)))) * state_cols +
                           state_col0 + i];
              acc = __fmaf_rn(c[t], hv, acc);
            }
          }
          if (flags & 1) normed[static_cast<size_t>(r) * normed_cols + normed_col0 + i] = h[j + kTaps - 1];
          out[static_cast<size_t>(r) * width + i] = bw::from_f<act_t>(__fadd_rn(h[j + kTaps - 1], acc));
        }
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
        if (row_keep[j] & 1) normed[static_cast<size_t>(r) * normed_cols + normed_col0 + i] = own;
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
  int slices = max(1, min((width + kConvThreads - 1) / kConvThreads, (sm_count() + groups - 1) / groups));
  const int chans = ((width + slices - 1) / slices + 31) / 32 * 32;
  slices = (width + chans - 1) / chans;
  auto go = [&](auto kernel) {
    bw::launch_pdl(kernel, dim3(groups, slices), dim3(kConvThreads), 0, stream, x, w, eps, taps_t, taps, state, state_cols,
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
