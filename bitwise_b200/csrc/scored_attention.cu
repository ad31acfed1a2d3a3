// Grouped-query softmax attention over paged keys and values with optional steps around the
// scores, and the kernels that prepare its operands.
//
//   qkv_prepare        per row and head: a short causal convolution over time on every channel of
//                      the projected q, k, v (inputs before the step's first row come from the
//                      request's state slot), a root-mean-square norm per head of q and k, the
//                      rotation of the leading entries of q and k (pair i = entries 2i, 2i + 1), q
//                      into the step's buffer, k and v into their pages
//   conv_state_update  the convolution's inputs of a request's last taps - 1 positions
//   scored_attention   s = (q . k) * scale; s <- cap * tanh(s / cap); s <- s - slope_h * (i - j);
//                      window; softmax with an optional extra one in the denominator; the values
//                      may be the keys themselves (no value pages)
//
// Everything after the projection is float32 in both precisions; only what is loaded and stored
// changes type. Keys are walked in tiles of 32 at fixed absolute positions, so what a query gets
// depends on its own keys only: not on the other rows of the step, nor on where a portion began.
#include "bw_act.cuh"
#include "bw_mma.cuh"

#include <math.h>

namespace {

// ---------------------------------------------------------------------------------------
// qkv_prepare. One block per row, a warp per head of q, k or v at a time; lane l holds the
// entries l, l + 32, ... of the head (up to kMaxE * 32).
constexpr int kMaxE = 8;
constexpr int kPrepWarps = 4;

struct PrepArgs {
  const float* u;            // [n, cols] projected rows: q heads, then k heads, then v heads
  int cols;
  int u_stride;              // floats between two rows of u (cols, or more where the rows are columns of a wider product)
  const float* bias;         // [cols] added to every projected row (also to rows read from the state), or null
  const float* vmix_src;     // [n, v_heads * vdim] values that this layer's values are mixed with, or null
  const float* vmix_lambda;  // one number: v <- (1 - lambda) v + lambda vmix_src
  float* v_keep;             // [n, v_heads * vdim]: the values as stored, kept in float32 for later layers, or null
  const float* conv_w;       // [cols, taps] or null
  const float* conv_wt;      // the same transposed, [taps, cols], for the kernel that reads four channels at a time
  int taps;
  const float* conv_state;   // [slots, taps - 1, cols] or null
  const float* q_norm;       // [dim] or null
  const float* k_norm;
  float eps;
  const float* cos_t;        // [positions, pairs] or null
  const float* sin_t;
  int pairs;
  const int* pos;
  const int* row_seq;
  const int* seq_row0;
  const int* seq_pos0;
  const int* seq_slot;
  const int* block_table;
  int max_blocks;
  act_t* kcache;             // [pages, kv_heads, page, dim]
  act_t* vcache;             // [pages, kv_heads, page, vdim] or null
  act_t* q_out;              // [n, heads * dim]
  int heads, kv_heads /* 0: nothing is stored */, v_heads, dim, vdim, page;
};

__global__ void __launch_bounds__(kPrepWarps * 32) qkv_prepare_kernel(const PrepArgs a) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = a.pos[r];
  const int seq = a.row_seq[r];
  const int row0 = a.seq_row0[seq];
  const int slot = a.conv_state ? a.seq_slot[seq] : 0;
  const int total = a.heads + a.kv_heads + a.v_heads;
  for (int hs = blockIdx.y * kPrepWarps + warp; hs < total; hs += kPrepWarps * gridDim.y) {
    int size, col0;
    const float* norm_w;
    bool turns;
    if (hs < a.heads) {
      size = a.dim, col0 = hs * a.dim, norm_w = a.q_norm, turns = true;
    } else if (hs < a.heads + a.kv_heads) {
      size = a.dim, col0 = hs * a.dim, norm_w = a.k_norm, turns = true;
    } else {
      size = a.vdim, col0 = (a.heads + a.kv_heads) * a.dim + (hs - a.heads - a.kv_heads) * a.vdim, norm_w = nullptr;
      turns = false;
    }
    float val[kMaxE];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxE; ++j) {
      const int e = lane + 32 * j;
      float v = 0.0f;
      if (e < size) {
        const int c = col0 + e;
        if (a.conv_w) {
          // y_t = sum_j w[c][j] * u_(t - taps + 1 + j), taps ascending; inputs before position 0 are zero
          for (int t = 0; t < a.taps; ++t) {
            const int back = a.taps - 1 - t;
            if (p - back < 0) continue;
            const int rr = r - back;
            float src = rr >= row0
                            ? a.u[static_cast<size_t>(rr) * a.u_stride + c]
                            : a.conv_state[(static_cast<size_t>(slot) * (a.taps - 1) + (a.taps - 1 - (row0 - rr))) * a.cols + c];
            if (a.bias) src = __fadd_rn(src, a.bias[c]);
            v = __fmaf_rn(a.conv_w[static_cast<size_t>(c) * a.taps + t], src, v);
          }
        } else {
          v = a.u[static_cast<size_t>(r) * a.u_stride + c];
          if (a.bias) v = __fadd_rn(v, a.bias[c]);
        }
        if (!turns && (a.vmix_src || a.v_keep)) {  // a value head (keys and queries turn or are normed; values neither)
          const size_t at = static_cast<size_t>(r) * a.v_heads * a.vdim + (hs - a.heads - a.kv_heads) * a.vdim + e;
          if (a.vmix_src) {
            const float lam = a.vmix_lambda[0];
            v = __fmaf_rn(lam, a.vmix_src[at], __fmul_rn(__fsub_rn(1.0f, lam), v));
          }
          if (a.v_keep) a.v_keep[at] = v;
        }
        ss = __fmaf_rn(v, v, ss);
      }
      val[j] = v;
    }
    if (norm_w) {
      const float inv = bw::rms_scale(bw::warp_sum(ss), size, a.eps);
#pragma unroll
      for (int j = 0; j < kMaxE; ++j) {
        const int e = lane + 32 * j;
        if (e < size) val[j] = bw::rms_apply(val[j], inv, norm_w[e]);
      }
    }
    if (turns && a.pairs > 0) {
#pragma unroll
      for (int j = 0; j < kMaxE; ++j) {
        const int e = lane + 32 * j;
        const float other = __shfl_xor_sync(0xffffffffu, val[j], 1);  // the partner of entry e is entry e ^ 1
        if (e < 2 * a.pairs && e < size) {
          const float c = a.cos_t[static_cast<size_t>(p) * a.pairs + (e >> 1)];
          const float s = a.sin_t[static_cast<size_t>(p) * a.pairs + (e >> 1)];
          val[j] = (e & 1) ? __fadd_rn(__fmul_rn(val[j], c), __fmul_rn(other, s))
                           : __fsub_rn(__fmul_rn(val[j], c), __fmul_rn(other, s));
        }
      }
    }
    act_t* dst;
    if (hs < a.heads) {
      dst = a.q_out + static_cast<size_t>(r) * a.heads * a.dim + hs * a.dim;
    } else {
      const int blk = a.block_table[static_cast<size_t>(seq) * a.max_blocks + p / a.page];
      if (hs < a.heads + a.kv_heads)
        dst = a.kcache + ((static_cast<size_t>(blk) * a.kv_heads + (hs - a.heads)) * a.page + p % a.page) * a.dim;
      else
        dst = a.vcache + ((static_cast<size_t>(blk) * a.v_heads + (hs - a.heads - a.kv_heads)) * a.page + p % a.page) * a.vdim;
    }
#pragma unroll
    for (int j = 0; j < kMaxE; ++j) {
      const int e = lane + 32 * j;
      if (e < size) dst[e] = bw::from_f<act_t>(val[j]);
    }
  }
}

// The same with four consecutive entries of a head per lane (head sizes and column counts that are
// multiples of 4): the projected rows, the state, the taps (transposed: [taps, cols]) and the norm
// weights are read 16 bytes at a time, a rotation's partners lie in one lane, and a lane stores its
// four results at once. Lane l holds entries 4 l .. 4 l + 3 and 128 + 4 l .. of the head.
#if BW_ACT_BF16
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
  uint2 w;
  w.x = bw::pack_bf16(v.x, v.y), w.y = bw::pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = w;
}
#else
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
#endif

__global__ void __launch_bounds__(kPrepWarps * 32) qkv_prepare_vec_kernel(const PrepArgs a) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = a.pos[r];
  const int seq = a.row_seq[r];
  const int row0 = a.seq_row0[seq];
  const int slot = a.conv_state ? a.seq_slot[seq] : 0;
  const int total = a.heads + a.kv_heads + a.v_heads;
  const float* urow = a.u + static_cast<size_t>(r) * a.u_stride;
  for (int hs = blockIdx.y * kPrepWarps + warp; hs < total; hs += kPrepWarps * gridDim.y) {
    int size, col0;
    const float* norm_w;
    bool turns;
    if (hs < a.heads + a.kv_heads) {
      size = a.dim, col0 = hs * a.dim, norm_w = hs < a.heads ? a.q_norm : a.k_norm, turns = true;
    } else {
      size = a.vdim, col0 = (a.heads + a.kv_heads) * a.dim + (hs - a.heads - a.kv_heads) * a.vdim, norm_w = nullptr;
      turns = false;
    }
    float4 val[2];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e0 = 4 * lane + 128 * j;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (e0 < size) {
        const int c = col0 + e0;
        if (a.conv_wt) {
          for (int t = 0; t < a.taps; ++t) {  // taps ascending, as in the kernel above
            const int back = a.taps - 1 - t;
            if (p - back < 0) continue;
            const int rr = r - back;
            const float* src = rr >= row0 ? urow - static_cast<size_t>(back) * a.u_stride + c
                                          : a.conv_state + (static_cast<size_t>(slot) * (a.taps - 1) + (a.taps - 1 - (row0 - rr))) * a.cols + c;
            float4 x = *reinterpret_cast<const float4*>(src);
            if (a.bias) {
              const float4 b = *reinterpret_cast<const float4*>(a.bias + c);
              x.x = __fadd_rn(x.x, b.x), x.y = __fadd_rn(x.y, b.y), x.z = __fadd_rn(x.z, b.z), x.w = __fadd_rn(x.w, b.w);
            }
            const float4 w = *reinterpret_cast<const float4*>(a.conv_wt + static_cast<size_t>(t) * a.cols + c);
            v.x = __fmaf_rn(w.x, x.x, v.x), v.y = __fmaf_rn(w.y, x.y, v.y), v.z = __fmaf_rn(w.z, x.z, v.z), v.w = __fmaf_rn(w.w, x.w, v.w);
          }
        } else {
          v = *reinterpret_cast<const float4*>(urow + c);
          if (a.bias) {
            const float4 b = *reinterpret_cast<const float4*>(a.bias + c);
            v.x = __fadd_rn(v.x, b.x), v.y = __fadd_rn(v.y, b.y), v.z = __fadd_rn(v.z, b.z), v.w = __fadd_rn(v.w, b.w);
          }
        }
        if (!turns && (a.vmix_src || a.v_keep)) {  // a value head
          const size_t at = static_cast<size_t>(r) * a.v_heads * a.vdim + (hs - a.heads - a.kv_heads) * a.vdim + e0;
          if (a.vmix_src) {
            const float lam = a.vmix_lambda[0], rest = __fsub_rn(1.0f, lam);
            const float4 f = *reinterpret_cast<const float4*>(a.vmix_src + at);
            v.x = __fmaf_rn(lam, f.x, __fmul_rn(rest, v.x)), v.y = __fmaf_rn(lam, f.y, __fmul_rn(rest, v.y));
            v.z = __fmaf_rn(lam, f.z, __fmul_rn(rest, v.z)), v.w = __fmaf_rn(lam, f.w, __fmul_rn(rest, v.w));
          }
          if (a.v_keep) *reinterpret_cast<float4*>(a.v_keep + at) = v;
        }
        ss = __fmaf_rn(v.x, v.x, ss), ss = __fmaf_rn(v.y, v.y, ss), ss = __fmaf_rn(v.z, v.z, ss), ss = __fmaf_rn(v.w, v.w, ss);
      }
      val[j] = v;
    }
    if (norm_w) {
      const float inv = bw::rms_scale(bw::warp_sum(ss), size, a.eps);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int e0 = 4 * lane + 128 * j;
        if (e0 < size) {
          const float4 w = *reinterpret_cast<const float4*>(norm_w + e0);
          val[j].x = bw::rms_apply(val[j].x, inv, w.x), val[j].y = bw::rms_apply(val[j].y, inv, w.y);
          val[j].z = bw::rms_apply(val[j].z, inv, w.z), val[j].w = bw::rms_apply(val[j].w, inv, w.w);
        }
      }
    }
    if (turns && a.pairs > 0) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int e0 = 4 * lane + 128 * j;
        if (e0 >= size) continue;
        const int i0 = e0 >> 1;
        const size_t at = static_cast<size_t>(p) * a.pairs;
        if (i0 < a.pairs) {
          const float c = a.cos_t[at + i0], s = a.sin_t[at + i0];
          const float x = val[j].x, y = val[j].y;
          val[j].x = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)), val[j].y = __fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s));
        }
        if (i0 + 1 < a.pairs) {
          const float c = a.cos_t[at + i0 + 1], s = a.sin_t[at + i0 + 1];
          const float x = val[j].z, y = val[j].w;
          val[j].z = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)), val[j].w = __fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s));
        }
      }
    }
    act_t* dst;
    if (hs < a.heads) {
      dst = a.q_out + static_cast<size_t>(r) * a.heads * a.dim + hs * a.dim;
    } else {
      const int blk = a.block_table[static_cast<size_t>(seq) * a.max_blocks + p / a.page];
      if (hs < a.heads + a.kv_heads)
        dst = a.kcache + ((static_cast<size_t>(blk) * a.kv_heads + (hs - a.heads)) * a.page + p % a.page) * a.dim;
      else
        dst = a.vcache + ((static_cast<size_t>(blk) * a.v_heads + (hs - a.heads - a.kv_heads)) * a.page + p % a.page) * a.vdim;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e0 = 4 * lane + 128 * j;
      if (e0 < size) store4(dst + e0, val[j]);
    }
  }
}

// state[slot][i] = the projected row of position end - (taps - 1) + i (i < taps - 1), `end` the
// request's length after this step: from the step's rows, from the old state, or zero before
// position 0. One thread per (sequence, channel) reads all it needs before it writes.
constexpr int kMaxTaps = 16;

__global__ void __launch_bounds__(128)
conv_state_update_kernel(const float* __restrict__ u, int u_stride, int cols, float* state, int taps, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                         const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot) {
  bw::pdl_enter();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int seq = tile_seq[t], row0 = tile_row0[t], cnt = tile_rows[t];
  const int pos0 = seq_pos0[seq];
  float* st = state + static_cast<size_t>(seq_slot[seq]) * (taps - 1) * cols + c;
  float keep[kMaxTaps];
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
    if (i >= taps - 1) break;
    const int p = pos0 + cnt - (taps - 1) + i;
    float v = 0.0f;
    if (p >= pos0)
      v = u[static_cast<size_t>(row0 + p - pos0) * u_stride + c];
    else if (p >= 0)
      v = st[static_cast<size_t>(p - pos0 + taps - 1) * cols];
    keep[i] = v;
  }
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
    if (i >= taps - 1) break;
    st[static_cast<size_t>(i) * cols] = keep[i];
  }
}

// ---------------------------------------------------------------------------------------
// Attention on the CUDA cores. A block takes one query tile (rows of one sequence at consecutive
// positions), one key/value head and up to `hb` of the query heads that read it; a warp works on
// one query (a row and a head) at a time, lane l on key l of the tile of 32: its score, the tile's
// maximum and sum over the warp, and the running (maximum, sum, weighted sum of values).
constexpr int kWarps = 8;
constexpr int kKeys = 32;
constexpr int kThreads = kWarps * 32;
constexpr int kQW = 4;  // queries per warp

struct ScoreArgs {
  float cap_exp;  // 2 * scale / softcap * log2(e): the exponent of the cap's exponential per unit of raw score
  float scale, softcap;
  int sink;
  const float* slopes;  // [heads] or null
  int window;
  const float* dist_a;  // [heads] or null: s <- s - dist_a[h] * ln(1 + dist_b[h] * (i - j))
  const float* dist_b;
  const float* sinks;   // [heads] or null: with `sink`, exp(sinks[h]) joins the denominator instead of exp(0)
  int keep_first;       // with a window: the keys j < keep_first stay visible to every later position
};

// What a query's head takes off a score by distance.
struct HeadBias {
  float slope, a, b;
};
__device__ __forceinline__ HeadBias head_bias(const ScoreArgs& sa, int h, bool ok) {
  HeadBias hb;
  hb.slope = sa.slopes && ok ? sa.slopes[h] : 0.0f;
  hb.a = sa.dist_a && ok ? sa.dist_a[h] : 0.0f;
  hb.b = sa.dist_a && ok ? sa.dist_b[h] : 0.0f;
  return hb;
}
// The first key a query at position pq sees inside its window (keys before keep_first are seen besides).
__device__ __forceinline__ bool key_seen(const ScoreArgs& sa, int pq, int lo, int kp) {
  return kp <= pq && (kp >= lo || kp < sa.keep_first);
}

#if BW_ACT_BF16
// The same on the serving precision's tensor-core path, where the scores come from bfloat16
// operands: tanh through the hardware's exponential, tanh(x) = 1 - 2 / (exp(2x) + 1) (relative
// error of a few 1e-7, against the 4e-3 of a bfloat16 operand).
__device__ __forceinline__ float modify_score_fast(float s, const ScoreArgs& sa, const HeadBias& hb, int pq, int kp) {
  if (sa.softcap > 0.0f) {
    // cap * tanh(x) = cap - 2 cap / (exp(2x) + 1), x = s * scale / cap; exp(2x) = 2^(s * cap_exp)
    const float e = bw::exp2_approx(__fmul_rn(s, sa.cap_exp));
    s = __fmaf_rn(__fmul_rn(-2.0f, sa.softcap), __fdividef(1.0f, __fadd_rn(e, 1.0f)), sa.softcap);
  } else {
    s = __fmul_rn(s, sa.scale);
  }
  if (sa.slopes) s = __fsub_rn(s, __fmul_rn(hb.slope, static_cast<float>(pq - kp)));
  if (sa.dist_a) s = __fsub_rn(s, __fmul_rn(hb.a, __logf(__fmaf_rn(hb.b, static_cast<float>(pq - kp), 1.0f))));
  return s;
}
#endif

__device__ __forceinline__ float modify_score(float s, const ScoreArgs& sa, const HeadBias& hb, int pq, int kp) {
  s = __fmul_rn(s, sa.scale);
  if (sa.softcap > 0.0f) s = __fmul_rn(sa.softcap, tanhf(__fdiv_rn(s, sa.softcap)));
  if (sa.slopes) s = __fsub_rn(s, __fmul_rn(hb.slope, static_cast<float>(pq - kp)));
  if (sa.dist_a) s = __fsub_rn(s, __fmul_rn(hb.a, log1pf(__fmul_rn(hb.b, static_cast<float>(pq - kp)))));
  return s;
}
// Key tiles of `tile` keys that a walk from `from` visits: with kept first keys the tiles that hold
// them, then the tiles from the window's first on; the tiles between are passed over.
__device__ __forceinline__ int skip_gap(int k0, int keep_end, int win_begin) {
  return (k0 >= keep_end && k0 < win_begin) ? win_begin : k0;
}

template <int ACC>
__global__ void __launch_bounds__(kThreads)
scored_attention_kernel(const act_t* __restrict__ q, int q_stride, const act_t* __restrict__ kcache,
                        const act_t* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                        const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                        const int* __restrict__ seq_row0, act_t* out, int o_stride, int heads, int kv_heads, int hb,
                        int dim, int vdim, int page, const ScoreArgs sa) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int ks = dim + 1;
  float* keys = sm;                                         // [32][dim + 1]
  float* vals = vcache ? keys + kKeys * ks : keys;          // [32][vdim], or the keys themselves
  const int vs = vcache ? vdim : ks;
  float* qs = keys + kKeys * ks + (vcache ? kKeys * vdim : 0);
  const int t = blockIdx.x, g = blockIdx.y;
  const int rep = heads / kv_heads;
  const int h0 = g * rep + blockIdx.z * hb;
  const int nh = min(hb, rep - blockIdx.z * hb);
  const int seq = tile_seq[t], row0 = tile_row0[t], rows = tile_rows[t];
  const int nq = rows * nh;
  const int p0 = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int qi = warp; qi < nq; qi += kWarps) {
    const act_t* src = q + static_cast<size_t>(row0 + qi / nh) * q_stride + (h0 + qi % nh) * dim;
    for (int d = lane; d < dim; d += 32) qs[qi * dim + d] = bw::to_f(src[d]);
  }
  float m[kQW], l[kQW], acc[kQW][ACC];
#pragma unroll
  for (int j = 0; j < kQW; ++j) {
    m[j] = -INFINITY, l[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[j][i] = 0.0f;
  }
  const int last = p0 + rows - 1;
  const int first = sa.window > 0 ? max(0, p0 - sa.window + 1) : 0;  // pages before it may be gone (kept first keys stay)
  const int keep = sa.window > 0 ? sa.keep_first : 0;
  const int keep_end = (keep + kKeys - 1) / kKeys * kKeys, win_begin = first / kKeys * kKeys;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  for (int k0 = skip_gap(0, keep_end, win_begin); k0 <= last; k0 = skip_gap(k0 + kKeys, keep_end, win_begin)) {
    __syncthreads();
    for (int kk = warp; kk < kKeys; kk += kWarps) {
      const int kp = k0 + kk;
      const bool have = kp <= last && (kp >= first || kp < keep);
      size_t at = 0;
      if (have) at = (static_cast<size_t>(bt[kp / page]) * kv_heads + g) * page + kp % page;
      for (int d = lane; d < dim; d += 32) keys[kk * ks + d] = have ? bw::to_f(kcache[at * dim + d]) : 0.0f;
      if (vcache)
        for (int d = lane; d < vdim; d += 32) vals[kk * vs + d] = have ? bw::to_f(vcache[at * vdim + d]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kQW; ++j) {
      const int qi = warp + kWarps * j;
      if (qi >= nq) continue;
      const int pq = p0 + qi / nh;
      const int lo = sa.window > 0 ? max(0, pq - sa.window + 1) : 0;
      if (k0 > pq || (k0 + kKeys <= lo && k0 >= keep)) continue;  // no key of the tile is seen: the state stays
      const int kp = k0 + lane;
      const float* qv = qs + qi * dim;
      const float* kv = keys + lane * ks;
      float s = 0.0f;
      for (int d = 0; d < dim; ++d) s = __fmaf_rn(qv[d], kv[d], s);
      s = modify_score(s, sa, head_bias(sa, h0 + qi % nh, true), pq, kp);
      const bool seen = key_seen(sa, pq, lo, kp);
      if (!seen) s = -INFINITY;
      const float mt = bw::warp_max(s);
      const float mn = fmaxf(m[j], mt);
      const float alpha = m[j] == -INFINITY ? 0.0f : expf(__fsub_rn(m[j], mn));
      const float pw = seen ? expf(__fsub_rn(s, mn)) : 0.0f;
      l[j] = __fmaf_rn(l[j], alpha, bw::warp_sum(pw));
#pragma unroll
      for (int i = 0; i < ACC; ++i) acc[j][i] = __fmul_rn(acc[j][i], alpha);
      for (int kk = 0; kk < kKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, pw, kk);
        if (pk == 0.0f) continue;
        const float* vrow = vals + kk * vs;
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
          const int d = i * 32 + lane;
          if (d < vdim) acc[j][i] = __fmaf_rn(pk, vrow[d], acc[j][i]);
        }
      }
      m[j] = mn;
    }
  }
#pragma unroll
  for (int j = 0; j < kQW; ++j) {
    const int qi = warp + kWarps * j;
    if (qi >= nq) continue;
    float den = l[j];
    if (sa.sink) den = __fadd_rn(den, expf(__fsub_rn(sa.sinks ? sa.sinks[h0 + qi % nh] : 0.0f, m[j])));  // the extra key (score 0 unless given)
    const float inv = __fdiv_rn(1.0f, den);
    act_t* dst = out + static_cast<size_t>(row0 + qi / nh) * o_stride + (h0 + qi % nh) * vdim;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int d = i * 32 + lane;
      if (d < vdim) dst[d] = bw::from_f<act_t>(__fmul_rn(acc[j][i], inv));
    }
  }
}

template <int ACC>
int launch_scored(dim3 grid, size_t smem, cudaStream_t stream, const act_t* q, int q_stride, const act_t* kcache,
                  const act_t* vcache, const int* block_table, int max_blocks, const int* tile_seq, const int* tile_row0,
                  const int* tile_rows, const int* seq_pos0, const int* seq_row0, act_t* out, int o_stride, int heads,
                  int kv_heads, int hb, int dim, int vdim, int page, const ScoreArgs& sa) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(scored_attention_kernel<ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("scored_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    allowed = smem;
  }
  bw::launch_pdl(scored_attention_kernel<ACC>, grid, dim3(kThreads), smem, stream, q, q_stride, kcache, vcache, block_table,
                 max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out, o_stride, heads, kv_heads, hb, dim,
                 vdim, page, sa);
  return bw::launch_status();
}


#if BW_ACT_BF16
// ---------------------------------------------------------------------------------------
// Attention on the tensor cores (bfloat16 operands, float32 accumulators; mma.sync m16n8k16).
// A block of four warps takes 64 stacked queries (rows of one query tile x the query heads of one
// key/value head), 16 per warp, and walks the keys in tiles of 32 at fixed absolute positions.
// Scores stay in the accumulators as float32: scale, cap, distance slope, mask, the running
// maximum and the weights exp(s - m) are formed there. The weights enter the second product as
// two bfloat16 parts (p = hi + lo), so the values are weighted with 16 bits of p. A query's
// result depends on its own keys and the fixed tiles only.
constexpr int kMmaWarps = 4;
constexpr int kMmaRows = 16 * kMmaWarps;
constexpr int kMmaKeys = 32;

template <int VD16 /* value size / 16 */>
__global__ void __launch_bounds__(kMmaWarps * 32)
scored_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ kcache,
                            const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                            const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                            const int* __restrict__ seq_row0, __nv_bfloat16* out, int o_stride, int heads, int kv_heads,
                            int hb, int dim, int page, const ScoreArgs sa, int span_tiles, int spans, float* partial) {
  bw::pdl_enter();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int vdim = VD16 * 16;
  constexpr int VT = VD16 * 2;  // accumulator tiles of 8 value columns
  const int kst = dim + 8;      // row strides in elements: 16 bytes more than a row, so that
  const int vst_own = vdim + 8; // ldmatrix reads eight rows from eight different banks
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [64][kst]
  __nv_bfloat16* ks_all = qs + kMmaRows * kst;                      // [2][32][kst]: the tile in use and the next
  __nv_bfloat16* vs_all = vcache ? ks_all + 2 * kMmaKeys * kst : ks_all;  // [2][32][vst]; the keys where values are keys
  const int vst = vcache ? vst_own : kst;
  const int t = blockIdx.x, g = blockIdx.y;
  const int rep = heads / kv_heads;
  const int zh = blockIdx.z / spans, span = blockIdx.z - zh * spans;  // the block's share of heads and of keys
  const int h0 = g * rep + zh * hb;
  const int nh = min(hb, rep - zh * hb);
  const int seq = tile_seq[t], row0 = tile_row0[t], rows = tile_rows[t];
  const int nq = rows * nh;
  const int p0 = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int dparts = dim >> 3, vparts = vdim >> 3;
  // this thread's two queries: stacked rows sa_ and sb_ of the block
  const int sr_a = warp * 16 + (lane >> 2), sr_b = sr_a + 8;
  const bool ok_a = sr_a < nq, ok_b = sr_b < nq;
  const int pq_a = p0 + (ok_a ? sr_a / nh : 0), pq_b = p0 + (ok_b ? sr_b / nh : 0);
  const int lo_a = sa.window > 0 ? max(0, pq_a - sa.window + 1) : 0, lo_b = sa.window > 0 ? max(0, pq_b - sa.window + 1) : 0;
  const HeadBias slope_a = head_bias(sa, h0 + sr_a % nh, ok_a), slope_b = head_bias(sa, h0 + sr_b % nh, ok_b);
  const int keep = sa.window > 0 ? sa.keep_first : 0;
  // the positions that this warp's queries span: tiles outside are skipped by the whole warp
  const int w_first = min(warp * 16, max(nq - 1, 0)) / nh, w_last = min(warp * 16 + 15, max(nq - 1, 0)) / nh;
  const int w_lo = sa.window > 0 ? max(0, p0 + w_first - sa.window + 1) : 0, w_hi = p0 + w_last;
  const bool warp_has_rows = warp * 16 < nq;
  const bool warp_full = warp * 16 + 15 < nq;  // all 16 stacked rows of the warp are queries
  const int w_seen_to = p0 + w_first;           // keys up to here are seen by every query of the warp ...
  const int w_seen_from = sa.window > 0 ? max(0, p0 + w_last - sa.window + 1) : 0;  // ... from here on
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
  float acc[VT][4];
#pragma unroll
  for (int j = 0; j < VT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
  const int last = p0 + rows - 1;
  const int first = sa.window > 0 ? max(0, p0 - sa.window + 1) : 0;  // pages before it may be gone (kept first keys stay)
  const int keep_end = (keep + kMmaKeys - 1) / kMmaKeys * kMmaKeys, win_begin = first / kMmaKeys * kMmaKeys;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  // With spans the block walks the key tiles span * span_tiles .. + span_tiles - 1 only (fixed
  // absolute positions again) and leaves a record for the merge instead of the result.
  int k_begin = skip_gap(0, keep_end, win_begin), k_end = last;
  if (span_tiles > 0) {
    k_begin = skip_gap(max(k_begin, span * span_tiles * kMmaKeys), keep_end, win_begin);
    k_end = min(k_end, (span + 1) * span_tiles * kMmaKeys - 1);
    if (k_begin > k_end) {
      // none of the block's queries reaches into this span: records that say so, nothing else
      for (int sr = tid; sr < nq; sr += kMmaWarps * 32) {
        float* rec = partial + ((static_cast<size_t>(row0 + sr / nh) * heads + h0 + sr % nh) * spans + span) * (vdim + 2);
        rec[0] = -INFINITY, rec[1] = 0.0f;
      }
      return;
    }
  }
  // the queries' rows (a block with keys to walk only)
  for (int c = tid; c < kMmaRows * dparts; c += kMmaWarps * 32) {
    const int sr = c / dparts, part = c - sr * dparts;
    const bool valid = sr < nq;
    const __nv_bfloat16* src = valid ? q + static_cast<size_t>(row0 + sr / nh) * q_stride + (h0 + sr % nh) * dim + part * 8 : q;
    bw::copy16_async(bw::smem_addr(qs + sr * kst + part * 8), src, valid);
  }
  bw::copies_commit();
  // The threads are laid over a tile's 16-byte parts as (key, part) with the parts rounded up to a
  // power of two, so that every thread keeps its part and steps through the keys.
  int pk = 1, pv = 1;
  while (pk < dparts) pk <<= 1;
  while (pv < vparts) pv <<= 1;
  const int part_k = tid & (pk - 1), kk0_k = tid / pk, kstep_k = max(1, kMmaWarps * 32 / pk);
  const int part_v = tid & (pv - 1), kk0_v = tid / pv, kstep_v = max(1, kMmaWarps * 32 / pv);
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;
  auto request_tile = [&](int k0, int buf) {
    __nv_bfloat16* kd = ks_all + buf * kMmaKeys * kst;
    __nv_bfloat16* vd = vs_all + buf * kMmaKeys * vst;
    // a thread copies one 16-byte part of the keys kk0, kk0 + kstep, ...: its part and first key are fixed
    for (int kk = kk0_k; kk < kMmaKeys; kk += kstep_k) {
      const int kp = k0 + kk;
      const bool have = kp <= last && (kp >= first || kp < keep) && part_k < dparts;
      const __nv_bfloat16* src = kcache;
      if (have) {
        const int blk = page_shift >= 0 ? kp >> page_shift : kp / page, slot = kp - blk * page;
        src = kcache + ((static_cast<size_t>(bt[blk]) * kv_heads + g) * page + slot) * dim + part_k * 8;
      }
      if (part_k < dparts) bw::copy16_async(bw::smem_addr(kd + kk * kst + part_k * 8), src, have);
    }
    if (vcache) {
      for (int kk = kk0_v; kk < kMmaKeys; kk += kstep_v) {
        const int kp = k0 + kk;
        const bool have = kp <= last && (kp >= first || kp < keep) && part_v < vparts;
        const __nv_bfloat16* src = vcache;
        if (have) {
          const int blk = page_shift >= 0 ? kp >> page_shift : kp / page, slot = kp - blk * page;
          src = vcache + ((static_cast<size_t>(bt[blk]) * kv_heads + g) * page + slot) * vdim + part_v * 8;
        }
        if (part_v < vparts) bw::copy16_async(bw::smem_addr(vd + kk * vst + part_v * 8), src, have);
      }
    }
    bw::copies_commit();
  };
  if (k_begin <= k_end) request_tile(k_begin, 0);
  for (int k0 = k_begin, buf = 0; k0 <= k_end; k0 = skip_gap(k0 + kMmaKeys, keep_end, win_begin), buf ^= 1) {
    // the next tile is requested while this one is used; its buffer was released by the
    // barrier at the end of the step before
    const int k_next = skip_gap(k0 + kMmaKeys, keep_end, win_begin);
    if (k_next <= k_end) {
      request_tile(k_next, buf ^ 1);
      bw::copies_wait<1>();
    } else {
      bw::copies_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* ks = ks_all + buf * kMmaKeys * kst;
    const __nv_bfloat16* vs = vs_all + buf * kMmaKeys * vst;
    if (warp_has_rows && k0 <= w_hi && (k0 + kMmaKeys > w_lo || k0 < keep)) {
    // scores of 16 queries x 32 keys
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
    for (int kk = 0; kk < dim; kk += 16) {
      uint32_t a[4], b[4];
      bw::ldsm4(a, bw::smem_addr(qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kst + kk + (lane >> 4) * 8));
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {  // 16 keys at a time
        bw::ldsm4(b, bw::smem_addr(ks + (jp * 16 + (lane >> 4) * 8 + (lane & 7)) * kst + kk + ((lane >> 3) & 1) * 8));
        bw::mma16816(sc[2 * jp], a, b[0], b[1]);
        bw::mma16816(sc[2 * jp + 1], a, b[2], b[3]);
      }
    }
    float mt_a = -INFINITY, mt_b = -INFINITY;
    // a tile that every query of the warp sees whole needs no mask
    const bool whole = warp_full && k0 + kMmaKeys - 1 <= w_seen_to && (k0 >= w_seen_from || k0 + kMmaKeys <= keep);
    if (whole) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kp = k0 + j * 8 + 2 * (lane & 3) + e;
          const float va = modify_score_fast(sc[j][e], sa, slope_a, pq_a, kp);
          const float vb = modify_score_fast(sc[j][2 + e], sa, slope_b, pq_b, kp);
          sc[j][e] = va, sc[j][2 + e] = vb;
          mt_a = fmaxf(mt_a, va), mt_b = fmaxf(mt_b, vb);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kp = k0 + j * 8 + 2 * (lane & 3) + e;
          float va = modify_score_fast(sc[j][e], sa, slope_a, pq_a, kp);
          float vb = modify_score_fast(sc[j][2 + e], sa, slope_b, pq_b, kp);
          if (!(ok_a && key_seen(sa, pq_a, lo_a, kp))) va = -INFINITY;
          if (!(ok_b && key_seen(sa, pq_b, lo_b, kp))) vb = -INFINITY;
          sc[j][e] = va, sc[j][2 + e] = vb;
          mt_a = fmaxf(mt_a, va), mt_b = fmaxf(mt_b, vb);
        }
      }
    }
    mt_a = fmaxf(mt_a, __shfl_xor_sync(0xffffffffu, mt_a, 1)), mt_a = fmaxf(mt_a, __shfl_xor_sync(0xffffffffu, mt_a, 2));
    mt_b = fmaxf(mt_b, __shfl_xor_sync(0xffffffffu, mt_b, 1)), mt_b = fmaxf(mt_b, __shfl_xor_sync(0xffffffffu, mt_b, 2));
    const float mn_a = fmaxf(m_a, mt_a), mn_b = fmaxf(m_b, mt_b);
    const float al_a = m_a == -INFINITY ? 0.0f : __expf(__fsub_rn(m_a, mn_a));
    const float al_b = m_b == -INFINITY ? 0.0f : __expf(__fsub_rn(m_b, mn_b));
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pa = sc[j][e] == -INFINITY ? 0.0f : __expf(__fsub_rn(sc[j][e], mn_a));
        const float pb = sc[j][2 + e] == -INFINITY ? 0.0f : __expf(__fsub_rn(sc[j][2 + e], mn_b));
        sc[j][e] = pa, sc[j][2 + e] = pb;
        sum_a = __fadd_rn(sum_a, pa), sum_b = __fadd_rn(sum_b, pb);
      }
    }
    l_a = __fmaf_rn(l_a, al_a, sum_a), l_b = __fmaf_rn(l_b, al_b, sum_b);  // this thread's share; joined at the end
    m_a = mn_a, m_b = mn_b;
    // (a maximum that stayed gives the factor exp(0) = 1 exactly: nothing to rescale then)
    if (__any_sync(0xffffffffu, al_a != 1.0f || al_b != 1.0f)) {
#pragma unroll
      for (int j = 0; j < VT; ++j) {
        acc[j][0] = __fmul_rn(acc[j][0], al_a), acc[j][1] = __fmul_rn(acc[j][1], al_a);
        acc[j][2] = __fmul_rn(acc[j][2], al_b), acc[j][3] = __fmul_rn(acc[j][3], al_b);
      }
    }
    // weighted values: 16 keys at a time, the weights as hi + lo
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      uint32_t hi[4], lw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x0 = sc[2 * kb + (i >> 1)][(i & 1) * 2], x1 = sc[2 * kb + (i >> 1)][(i & 1) * 2 + 1];
        const __nv_bfloat16 h0b = __float2bfloat16_rn(x0), h1b = __float2bfloat16_rn(x1);
        hi[i] = bw::pack_bf16(x0, x1);
        lw[i] = bw::pack_bf16(__fsub_rn(x0, __bfloat162float(h0b)), __fsub_rn(x1, __bfloat162float(h1b)));
      }
#pragma unroll
      for (int jp = 0; jp < VD16; ++jp) {  // 16 value columns at a time
        uint32_t b[4];
        bw::ldsm4_trans(b, bw::smem_addr(vs + (kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * vst + jp * 16 + (lane >> 4) * 8));
        bw::mma16816(acc[2 * jp], hi, b[0], b[1]);
        bw::mma16816(acc[2 * jp], lw, b[0], b[1]);
        bw::mma16816(acc[2 * jp + 1], hi, b[2], b[3]);
        bw::mma16816(acc[2 * jp + 1], lw, b[2], b[3]);
      }
    }
    }
    __syncthreads();  // every warp has used the tile: its buffer may be filled again
  }
  bw::copies_wait<0>();  // (a block without a key tile has not waited for its queries' copies yet)
  l_a = __fadd_rn(l_a, __shfl_xor_sync(0xffffffffu, l_a, 1)), l_a = __fadd_rn(l_a, __shfl_xor_sync(0xffffffffu, l_a, 2));
  l_b = __fadd_rn(l_b, __shfl_xor_sync(0xffffffffu, l_b, 1)), l_b = __fadd_rn(l_b, __shfl_xor_sync(0xffffffffu, l_b, 2));
  if (span_tiles > 0) {
    // the span's record per query: maximum, sum, weighted values relative to that maximum
    const int colp = 2 * (lane & 3);
    if (ok_a) {
      float* rec = partial + ((static_cast<size_t>(row0 + sr_a / nh) * heads + h0 + sr_a % nh) * spans + span) * (vdim + 2);
      if ((lane & 3) == 0) rec[0] = m_a, rec[1] = l_a;
#pragma unroll
      for (int j = 0; j < VT; ++j) rec[2 + j * 8 + colp] = acc[j][0], rec[2 + j * 8 + colp + 1] = acc[j][1];
    }
    if (ok_b) {
      float* rec = partial + ((static_cast<size_t>(row0 + sr_b / nh) * heads + h0 + sr_b % nh) * spans + span) * (vdim + 2);
      if ((lane & 3) == 0) rec[0] = m_b, rec[1] = l_b;
#pragma unroll
      for (int j = 0; j < VT; ++j) rec[2 + j * 8 + colp] = acc[j][2], rec[2 + j * 8 + colp + 1] = acc[j][3];
    }
    return;
  }
  if (sa.sink) {  // the extra key (score 0 unless the head has a number of its own)
    const float sk_a = sa.sinks && ok_a ? sa.sinks[h0 + sr_a % nh] : 0.0f, sk_b = sa.sinks && ok_b ? sa.sinks[h0 + sr_b % nh] : 0.0f;
    l_a = __fadd_rn(l_a, expf(__fsub_rn(sk_a, m_a))), l_b = __fadd_rn(l_b, expf(__fsub_rn(sk_b, m_b)));
  }
  const float inv_a = __fdiv_rn(1.0f, l_a), inv_b = __fdiv_rn(1.0f, l_b);
  const int col = 2 * (lane & 3);
  if (ok_a) {
    __nv_bfloat16* dst = out + static_cast<size_t>(row0 + sr_a / nh) * o_stride + (h0 + sr_a % nh) * vdim + col;
#pragma unroll
    for (int j = 0; j < VT; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(__fmul_rn(acc[j][0], inv_a), __fmul_rn(acc[j][1], inv_a));
  }
  if (ok_b) {
    __nv_bfloat16* dst = out + static_cast<size_t>(row0 + sr_b / nh) * o_stride + (h0 + sr_b % nh) * vdim + col;
#pragma unroll
    for (int j = 0; j < VT; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(__fmul_rn(acc[j][2], inv_b), __fmul_rn(acc[j][3], inv_b));
  }
}

// The spans' records of a query joined in ascending order of the spans: a warp per query.
__global__ void __launch_bounds__(128)
scored_attention_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* out, int o_stride, int queries, int heads,
                              int vdim, int spans, int sink, const float* __restrict__ sinks) {
  bw::pdl_enter();
  const int qi = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (qi >= queries) return;
  const float* rec = partial + static_cast<size_t>(qi) * spans * (vdim + 2);
  float m = -INFINITY;
  for (int s = 0; s < spans; ++s) m = fmaxf(m, rec[static_cast<size_t>(s) * (vdim + 2)]);
  float l = 0.0f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int s = 0; s < spans; ++s) {
    const float* r = rec + static_cast<size_t>(s) * (vdim + 2);
    if (r[0] == -INFINITY) continue;  // a span in which the query saw no key
    const float f = expf(__fsub_rn(r[0], m));
    l = __fmaf_rn(r[1], f, l);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = i * 32 + lane;
      if (d < vdim) acc[i] = __fmaf_rn(r[2 + d], f, acc[i]);
    }
  }
  if (sink) l = __fadd_rn(l, expf(__fsub_rn(sinks ? sinks[qi % heads] : 0.0f, m)));
  const float inv = __fdiv_rn(1.0f, l);
  __nv_bfloat16* dst = out + static_cast<size_t>(qi / heads) * o_stride + (qi % heads) * vdim;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = i * 32 + lane;
    if (d < vdim) dst[d] = __float2bfloat16_rn(__fmul_rn(acc[i], inv));
  }
}

template <int VD16>
int launch_scored_mma(dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* q, int q_stride,
                      const __nv_bfloat16* kcache, const __nv_bfloat16* vcache, const int* block_table, int max_blocks,
                      const int* tile_seq, const int* tile_row0, const int* tile_rows, const int* seq_pos0,
                      const int* seq_row0, __nv_bfloat16* out, int o_stride, int heads, int kv_heads, int hb, int dim,
                      int page, const ScoreArgs& sa, int span_tiles, int spans, float* partial) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(scored_attention_mma_kernel<VD16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("scored_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    allowed = smem;
  }
  bw::launch_pdl(scored_attention_mma_kernel<VD16>, grid, dim3(kMmaWarps * 32), smem, stream, q, q_stride, kcache, vcache,
                 block_table, max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out, o_stride, heads, kv_heads,
                 hb, dim, page, sa, span_tiles, spans, partial);
  return bw::launch_status();
}

bool g_force_plain = false;
constexpr int kSpanTiles = 8;  // key tiles per span: 256 keys, whatever the step
#endif  // BW_ACT_BF16

}  // namespace

// Rows of one sequence per query tile for `group` query heads on a key/value head.
BW_API int BW_FN(scored_attention_tile_rows)(int group) {
  const int hb = group < kWarps * kQW ? group : kWarps * kQW;
  return (kWarps * kQW) / (hb > 0 ? hb : 1);
}

BW_API int BW_FN(qkv_prepare)(const float* u, int cols, const float* conv_w, const float* conv_wt, int taps,
                              const float* conv_state,
                              const float* q_norm, const float* k_norm, float eps, const float* cos_t, const float* sin_t,
                              int pairs, const int* pos, const int* row_seq, const int* seq_row0, const int* seq_pos0,
                              const int* seq_slot, const int* block_table, int max_blocks, void* kcache, void* vcache,
                              void* q_out, int n, int heads, int kv_heads, int dim, int vdim, int page,
                              const float* bias, const float* vmix_src, const float* vmix_lambda, float* v_keep,
                              int u_stride, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (u_stride < cols) {
    bw::set_error("qkv_prepare: rows %d floats apart do not hold %d columns", u_stride, cols);
    return -1;
  }
  if (dim > kMaxE * 32 || vdim > kMaxE * 32) {
    bw::set_error("qkv_prepare: head sizes %d / %d (up to %d)", dim, vdim, kMaxE * 32);
    return -1;
  }
  if (conv_w && taps > 1 && !conv_state) {
    bw::set_error("qkv_prepare: a convolution of %d taps needs the requests' state", taps);
    return -1;
  }
  PrepArgs a;
  a.bias = bias, a.vmix_src = vmix_src, a.vmix_lambda = vmix_lambda, a.v_keep = v_keep;
  a.u = u, a.cols = cols, a.u_stride = u_stride, a.conv_w = conv_w, a.conv_wt = conv_w ? conv_wt : nullptr, a.taps = taps;
  a.conv_state = taps > 1 ? conv_state : nullptr;
  a.q_norm = q_norm, a.k_norm = k_norm, a.eps = eps, a.cos_t = cos_t, a.sin_t = sin_t, a.pairs = cos_t ? pairs : 0;
  a.pos = pos, a.row_seq = row_seq, a.seq_row0 = seq_row0, a.seq_pos0 = seq_pos0, a.seq_slot = seq_slot;
  a.block_table = block_table, a.max_blocks = max_blocks;
  a.kcache = static_cast<act_t*>(kcache), a.vcache = static_cast<act_t*>(vcache), a.q_out = static_cast<act_t*>(q_out);
  a.heads = heads, a.kv_heads = kv_heads, a.v_heads = vcache ? kv_heads : 0, a.dim = dim, a.vdim = vdim, a.page = page;
  const int total = heads + kv_heads + a.v_heads;
  // four entries per lane where every head and row starts on 16 bytes (and the taps came transposed)
  const bool by_four = dim % 4 == 0 && vdim % 4 == 0 && cols % 4 == 0 && u_stride % 4 == 0 && (!conv_w || conv_wt) &&
                       ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(conv_state) |
                         reinterpret_cast<uintptr_t>(conv_wt) | reinterpret_cast<uintptr_t>(q_norm) |
                         reinterpret_cast<uintptr_t>(k_norm) | reinterpret_cast<uintptr_t>(bias) |
                         reinterpret_cast<uintptr_t>(vmix_src) | reinterpret_cast<uintptr_t>(v_keep)) & 15) == 0;
  if (by_four)
    bw::launch_pdl(qkv_prepare_vec_kernel, dim3(n, (total + kPrepWarps - 1) / kPrepWarps), dim3(kPrepWarps * 32), 0, stream, a);
  else
    bw::launch_pdl(qkv_prepare_kernel, dim3(n, (total + kPrepWarps - 1) / kPrepWarps), dim3(kPrepWarps * 32), 0, stream, a);
  return bw::launch_status();
}

// u_stride: floats between two rows of u (at least cols).
BW_API int BW_FN(conv_state_update)(const float* u, int cols, float* state, int taps, const int* tile_seq,
                                    const int* tile_row0, const int* tile_rows, int tiles, const int* seq_pos0,
                                    const int* seq_slot, int u_stride, cudaStream_t stream) {
  if (tiles <= 0 || taps <= 1) return 0;
  if (u_stride < cols) {
    bw::set_error("conv_state_update: rows %d floats apart do not hold %d columns", u_stride, cols);
    return -1;
  }
  if (taps - 1 > kMaxTaps) {
    bw::set_error("conv_state_update: %d taps (up to %d)", taps, kMaxTaps + 1);
    return -1;
  }
  bw::launch_pdl(conv_state_update_kernel, dim3(tiles, (cols + 127) / 128), dim3(128), 0, stream, u, u_stride, cols, state, taps,
                 tile_seq, tile_row0, tile_rows, seq_pos0, seq_slot);
  return bw::launch_status();
}

BW_API int BW_FN(scored_attention)(const void* q, int q_stride, const void* kcache, const void* vcache,
                                   const int* block_table, int max_blocks, const int* tile_seq, const int* tile_row0,
                                   const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_row0, void* out,
                                   int o_stride, int heads, int kv_heads, int dim, int vdim, int page, float scale,
                                   float softcap, int sink, const float* slopes, int window, const float* dist_a,
                                   const float* dist_b, const float* sinks, int keep_first, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads) {
    bw::set_error("scored_attention: %d heads on %d key/value heads", heads, kv_heads);
    return -1;
  }
  const int acc = (vdim + 31) / 32;
  if (acc > 8) {
    bw::set_error("scored_attention: value size %d (up to 256)", vdim);
    return -1;
  }
  const int rep = heads / kv_heads;
  const int hb = rep < kWarps * kQW ? rep : kWarps * kQW;
  const size_t smem = (static_cast<size_t>(kKeys) * (dim + 1) + (vcache ? static_cast<size_t>(kKeys) * vdim : 0) +
                       static_cast<size_t>(kWarps * kQW) * dim) * sizeof(float);
  if (smem > 200 * 1024) {
    bw::set_error("scored_attention: head sizes %d / %d need %zu bytes of shared memory", dim, vdim, smem);
    return -1;
  }
  ScoreArgs sa;
  sa.scale = scale, sa.softcap = softcap, sa.sink = sink, sa.slopes = slopes, sa.window = window;
  sa.dist_a = dist_a, sa.dist_b = dist_a ? dist_b : nullptr, sa.sinks = sinks, sa.keep_first = window > 0 ? keep_first : 0;
  sa.cap_exp = 0.0f;  // (the tensor-core kernel's)
  const dim3 grid(tiles, kv_heads, (rep + hb - 1) / hb);
#define BW_SCORED(A)                                                                                                      \
  case A:                                                                                                                 \
    return launch_scored<A>(grid, smem, stream, static_cast<const act_t*>(q), q_stride, static_cast<const act_t*>(kcache), \
                            static_cast<const act_t*>(vcache), block_table, max_blocks, tile_seq, tile_row0, tile_rows,   \
                            seq_pos0, seq_row0, static_cast<act_t*>(out), o_stride, heads, kv_heads, hb, dim, vdim, page, \
                            sa);
  switch (acc) {
    BW_SCORED(1) BW_SCORED(2) BW_SCORED(3) BW_SCORED(4) BW_SCORED(5) BW_SCORED(6) BW_SCORED(7) BW_SCORED(8)
  }
#undef BW_SCORED
  return -1;
}

#if BW_ACT_BF16
// Tests: keep attention on the CUDA-core kernel also where the tensor-core kernel takes the shape.
BW_API int bw_bf16_scored_attention_force_plain(int on) {
  g_force_plain = on != 0;
  return 0;
}

// Rows of one sequence per query tile of the tensor-core kernel, 0 where it does not take the
// shape: key size a multiple of 16, value size 16 .. 128 in steps of 16, or 256.
BW_API int bw_bf16_scored_attention_mma_tile_rows(int group, int dim, int vdim) {
  if (g_force_plain || dim % 16 || vdim % 16 || dim > 256 || !(vdim <= 128 || vdim == 256)) return 0;
  const int hb = group < kMmaRows ? group : kMmaRows;
  return kMmaRows / (hb > 0 ? hb : 1);
}

BW_API int bw_bf16_scored_attention_mma(const void* q, int q_stride, const void* kcache, const void* vcache,
                                        const int* block_table, int max_blocks, const int* tile_seq, const int* tile_row0,
                                        const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_row0, void* out,
                                        int o_stride, int heads, int kv_heads, int dim, int vdim, int page, float scale,
                                        float softcap, int sink, const float* slopes, int window, int n, int spans,
                                        float* partial, const float* dist_a, const float* dist_b, const float* sinks,
                                        int keep_first, cudaStream_t stream) {
  // spans > 1 (`partial` holding n * heads * spans * (vdim + 2) floats): every query's keys are spread
  // over blocks of kSpanTiles key tiles each, at fixed absolute positions, and a second kernel joins
  // the spans' records in ascending order.
  if (tiles <= 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || !bw_bf16_scored_attention_mma_tile_rows(heads / kv_heads, dim, vdim)) {
    bw::set_error("scored_attention (tensor cores): %d heads on %d, sizes %d / %d", heads, kv_heads, dim, vdim);
    return -1;
  }
  const int rep = heads / kv_heads;
  const int hb = rep < kMmaRows ? rep : kMmaRows;
  const size_t smem = (static_cast<size_t>(kMmaRows + 2 * kMmaKeys) * (dim + 8) +
                       (vcache ? static_cast<size_t>(2 * kMmaKeys) * (vdim + 8) : 0)) * sizeof(__nv_bfloat16);
  ScoreArgs sa;
  sa.scale = scale, sa.softcap = softcap, sa.sink = sink, sa.slopes = slopes, sa.window = window;
  sa.dist_a = dist_a, sa.dist_b = dist_a ? dist_b : nullptr, sa.sinks = sinks, sa.keep_first = window > 0 ? keep_first : 0;
  sa.cap_exp = softcap > 0.0f ? 2.0f * scale / softcap * 1.4426950408889634f : 0.0f;
  const bool split = spans > 1 && partial != nullptr;
  if (!split) spans = 1;
  const dim3 grid(tiles, kv_heads, (rep + hb - 1) / hb * spans);
  typedef const __nv_bfloat16* in_t;
  int rc = -1;
#define BW_SCORED_MMA(V)                                                                                                   \
  case V:                                                                                                                  \
    rc = launch_scored_mma<V>(grid, smem, stream, static_cast<in_t>(q), q_stride, static_cast<in_t>(kcache),               \
                              static_cast<in_t>(vcache), block_table, max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, \
                              seq_row0, static_cast<__nv_bfloat16*>(out), o_stride, heads, kv_heads, hb, dim, page, sa,     \
                              split ? kSpanTiles : 0, spans, partial);                                                      \
    break;
  switch (vdim / 16) {
    BW_SCORED_MMA(1) BW_SCORED_MMA(2) BW_SCORED_MMA(3) BW_SCORED_MMA(4) BW_SCORED_MMA(5) BW_SCORED_MMA(6) BW_SCORED_MMA(7)
    BW_SCORED_MMA(8) BW_SCORED_MMA(16)
  }
#undef BW_SCORED_MMA
  if (rc != 0 || !split) return rc;
  bw::launch_pdl(scored_attention_merge_kernel, dim3((n * heads + 3) / 4), dim3(128), 0, stream,
                 static_cast<const float*>(partial), static_cast<__nv_bfloat16*>(out), o_stride, n * heads, heads, vdim, spans, sink, sinks);
  return bw::launch_status();
}

// Spans that a step of single rows with contexts of up to max_keys keys is spread over.
BW_API int bw_bf16_scored_attention_spans(int max_keys) {
  const int per = kSpanTiles * kMmaKeys;
  return (max_keys + per - 1) / per;
}
#endif  // BW_ACT_BF16
