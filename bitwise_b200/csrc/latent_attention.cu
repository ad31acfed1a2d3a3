// Attention over a latent cache. A token keeps one vector of `rank` + `rot_dim` numbers for all
// heads: a normed latent c, from which every head's keys and values are linear maps, and one
// rotated key part that the heads share. With the heads' key maps folded into the queries
// (q' = W_uk^T q, done by the caller as a product per head) a head's score against a cached
// token is one dot product of rank + rot_dim terms against that vector, and what attention
// returns per head is the weighted sum of latents, which the caller maps to values afterwards:
// the cache is read once for all heads and never expanded.
//
// Kernels: the store (root-mean-square norm of the latent, rotation of the shared key part,
// write into the page), the rotation of the queries' rotated parts, attention for query tiles
// (prompt portions and steps of few rows alike), and attention split over the keys for steps of
// single rows, with its merge; each attention once on the CUDA cores (both precisions) and once
// on the tensor cores (bfloat16). Scores, softmax weights, sums and rotations are float32 in
// both precisions.
#include "bw_act.cuh"
#include "bw_mma.cuh"

#include <math.h>

namespace {

// ---------------------------------------------------------------------------------------
// The rotation of pair i (entries 2i and 2i + 1 of a vector) by the table row of the
// position: (u, v) -> (u cos - v sin, v cos + u sin). `pairs` pairs are turned, entries
// from 2 * pairs on pass unchanged. In the half layout (`half_layout` != 0) pair i is made of
// entries i and i + pairs instead.
__device__ __forceinline__ void turn(float u, float v, float c, float s, float& ru, float& rv) {
  ru = __fsub_rn(__fmul_rn(u, c), __fmul_rn(v, s));
  rv = __fadd_rn(__fmul_rn(v, c), __fmul_rn(u, s));
}

// Entry i of the vector `src` after the rotation in the half layout: entry i < pairs is the first of its
// pair and entry i + pairs the second; entries from 2 * pairs on pass unchanged. `load` reads an entry
// as float.
template <typename Load>
__device__ __forceinline__ float turned_half(Load load, int i, int pairs, const float* __restrict__ cos_row,
                                             const float* __restrict__ sin_row) {
  const float self = load(i);
  if (i >= 2 * pairs) return self;
  const int j = i < pairs ? i : i - pairs;
  const float c = cos_row[j], s = sin_row[j];
  return i < pairs ? __fsub_rn(__fmul_rn(self, c), __fmul_rn(load(i + pairs), s))
                   : __fadd_rn(__fmul_rn(self, c), __fmul_rn(load(i - pairs), s));
}

// One block per row: d = the row of the down projection (float32, rank + rot_dim wide).
// cache[page][slot] = [ d[:rank] / sqrt(mean(d[:rank]^2) + eps) * w | turn(d[rank:]) ].
// With q_out the q_rank numbers that follow in the row are the queries' latent before its norm:
// q_out[row] = them / sqrt(mean(them^2) + eps) * q_w, so that one kernel serves both latents of a row
// where one product formed both.
__global__ void __launch_bounds__(128)
latent_store_kernel(const float* __restrict__ d, int d_stride, const float* __restrict__ w, float eps,
                    const int* __restrict__ pos, const int* __restrict__ row_seq, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int pairs, const int* __restrict__ block_table, int max_blocks,
                    act_t* cache, int rank, int rot_dim, int page, int half_layout, const float* __restrict__ q_w,
                    int q_rank, act_t* q_out) {
  bw::pdl_enter();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* dr = d + static_cast<size_t>(r) * d_stride;
  if (q_out) {
    const float* qr = dr + rank + rot_dim;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq = __fmaf_rn(qr[i], qr[i], sq);
    const float qinv = bw::rms_scale(bw::block_sum(sq, red), q_rank, eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      q_out[static_cast<size_t>(r) * q_rank + i] = bw::from_f<act_t>(bw::rms_apply(qr[i], qinv, q_w[i]));
  }
  const int p = pos[r];
  const int blk = block_table[static_cast<size_t>(row_seq[r]) * max_blocks + p / page];
  act_t* dst = cache + (static_cast<size_t>(blk) * page + p % page) * (rank + rot_dim);
  float ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = __fmaf_rn(dr[i], dr[i], ss);
  const float inv = bw::rms_scale(bw::block_sum(ss, red), rank, eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = bw::from_f<act_t>(bw::rms_apply(dr[i], inv, w[i]));
  const float* kr = dr + rank;
  if (half_layout) {
    const float* cr = cos_t + static_cast<size_t>(p) * pairs;
    const float* sr = sin_t + static_cast<size_t>(p) * pairs;
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x)
      dst[rank + i] = bw::from_f<act_t>(turned_half([&](int e) { return kr[e]; }, i, pairs, cr, sr));
    return;
  }
  for (int i = threadIdx.x; i < (rot_dim + 1) / 2; i += blockDim.x) {
    const float u = kr[2 * i];
    if (2 * i + 1 >= rot_dim) {  // an odd last entry has no partner
      dst[rank + 2 * i] = bw::from_f<act_t>(u);
      continue;
    }
    const float v = kr[2 * i + 1];
    float ru = u, rv = v;
    if (i < pairs) turn(u, v, cos_t[static_cast<size_t>(p) * pairs + i], sin_t[static_cast<size_t>(p) * pairs + i], ru, rv);
    dst[rank + 2 * i] = bw::from_f<act_t>(ru);
    dst[rank + 2 * i + 1] = bw::from_f<act_t>(rv);
  }
}

// The rotated part of every head's query: `rot_dim` entries at q[row][h * head_stride + offset],
// turned and written to out[row][h * out_head_stride + out_offset]. One block per row; a thread
// takes a pair of one head.
__global__ void __launch_bounds__(128)
rotate_heads_kernel(const act_t* __restrict__ q, int q_stride, int head_stride, int offset, act_t* out, int o_stride,
                    int out_head_stride, int out_offset, int heads, int rot_dim, int pairs, const int* __restrict__ pos,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half_layout) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int p = pos[r];
  if (half_layout) {
    const float* cr = cos_t + static_cast<size_t>(p) * pairs;
    const float* sr = sin_t + static_cast<size_t>(p) * pairs;
    for (int item = threadIdx.x; item < heads * rot_dim; item += blockDim.x) {
      const int h = item / rot_dim, i = item - h * rot_dim;
      const act_t* src = q + static_cast<size_t>(r) * q_stride + h * head_stride + offset;
      out[static_cast<size_t>(r) * o_stride + h * out_head_stride + out_offset + i] =
          bw::from_f<act_t>(turned_half([&](int e) { return bw::to_f(src[e]); }, i, pairs, cr, sr));
    }
    return;
  }
  const int half = (rot_dim + 1) / 2;
  for (int item = threadIdx.x; item < heads * half; item += blockDim.x) {
    const int h = item / half, i = item - h * half;
    const act_t* src = q + static_cast<size_t>(r) * q_stride + h * head_stride + offset;
    act_t* dst = out + static_cast<size_t>(r) * o_stride + h * out_head_stride + out_offset;
    const float u = bw::to_f(src[2 * i]);
    if (2 * i + 1 >= rot_dim) {
      dst[2 * i] = bw::from_f<act_t>(u);
      continue;
    }
    const float v = bw::to_f(src[2 * i + 1]);
    float ru = u, rv = v;
    if (i < pairs) turn(u, v, cos_t[static_cast<size_t>(p) * pairs + i], sin_t[static_cast<size_t>(p) * pairs + i], ru, rv);
    dst[2 * i] = bw::from_f<act_t>(ru);
    dst[2 * i + 1] = bw::from_f<act_t>(rv);
  }
}

// ---------------------------------------------------------------------------------------
// Attention. Keys are walked in tiles of 32 at fixed absolute positions (tile t holds positions
// 32 t .. 32 t + 31); lane l of a warp owns key l of the tile. A warp works on one query (a row
// and a head) at a time: the score of its key, the tile's maximum and sum over the warp, and
// the running (maximum, sum, weighted sum of latents) of the query, rescaled tile by tile. What
// a query gets depends on its own keys and on the fixed tiles only: not on the other queries of
// the block, nor on where the block started. A tile in which a query sees no key leaves its
// state untouched.
constexpr int kWarps = 8;
constexpr int kKeys = 32;
constexpr int kThreads = kWarps * 32;

// A sink: a learned logit per head that joins the softmax's denominator once, with no key and no
// value. `l` is the sum of exp(s - m) over the keys seen; `sinks` null: the sum stays as it is.
__device__ __forceinline__ float with_sink(float l, float m, const float* __restrict__ sinks, int h) {
  return sinks ? __fadd_rn(l, expf(__fsub_rn(sinks[h], m))) : l;
}

// One tile of keys in shared memory (`keys`, rows of `ks` floats) against the query `qv`
// (`dk` floats in shared memory) of position `pq`: updates m, l and acc (entry i of acc is
// latent dimension 32 i + lane).
template <int ACC>
__device__ __forceinline__ void attend_tile(const float* keys, int ks, const float* qv, int dk, int rank, int k0,
                                            int lo, int pq, float scale, int lane, float& m, float& l, float* acc) {
  const int kp = k0 + lane;
  const float* kv = keys + lane * ks;
  float s = 0.0f;
  for (int d = 0; d < dk; ++d) s = __fmaf_rn(qv[d], kv[d], s);
  s = __fmul_rn(s, scale);
  const bool seen = kp <= pq && kp >= lo;
  if (!seen) s = -INFINITY;
  const float mt = bw::warp_max(s);
  if (mt == -INFINITY) return;  // the same for all lanes
  const float mn = fmaxf(m, mt);
  const float alpha = m == -INFINITY ? 0.0f : expf(__fsub_rn(m, mn));
  const float p = seen ? expf(__fsub_rn(s, mn)) : 0.0f;
  l = __fmaf_rn(l, alpha, bw::warp_sum(p));
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = __fmul_rn(acc[i], alpha);
  for (int kk = 0; kk < kKeys; ++kk) {
    const float pk = __shfl_sync(0xffffffffu, p, kk);
    if (pk == 0.0f) continue;
    const float* vrow = keys + kk * ks;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int d = i * 32 + lane;
      if (d < rank) acc[i] = __fmaf_rn(pk, vrow[d], acc[i]);
    }
  }
  m = mn;
}

// Loads the keys k0 .. k0 + 31 of one sequence (those up to `last`) into shared memory.
__device__ __forceinline__ void load_keys(float* keys, int ks, const act_t* __restrict__ cache, const int* __restrict__ bt,
                                          int page, int dk, int k0, int last, int warp, int lane) {
  for (int kk = warp; kk < kKeys; kk += kWarps) {
    const int kp = k0 + kk;
    float* dst = keys + kk * ks;
    if (kp <= last) {
      const act_t* src = cache + (static_cast<size_t>(bt[kp / page]) * page + kp % page) * dk;
      for (int d = lane; d < dk; d += 32) dst[d] = bw::to_f(src[d]);
    } else {
      for (int d = lane; d < dk; d += 32) dst[d] = 0.0f;
    }
  }
}

// Query tiles: a block takes the rows of one tile (rows of one sequence, consecutive positions)
// and `hb` heads from h0 = blockIdx.y * hb on; its queries are (row, head) pairs, at most
// kWarps * QW of them, query i on warp i % kWarps.
template <int ACC, int QW>
__global__ void __launch_bounds__(kThreads)
latent_attention_kernel(const act_t* __restrict__ q, int q_stride, const act_t* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tile_seq,
                        const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                        const int* __restrict__ seq_pos0, const int* __restrict__ seq_row0, act_t* out, int o_stride,
                        int heads, int hb, int rank, int rot_dim, int page, int window, float scale,
                        const float* __restrict__ sinks) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int dk = rank + rot_dim, ks = dk + 1;
  float* keys = sm;
  float* qs = sm + kKeys * ks;
  const int t = blockIdx.x;
  const int seq = tile_seq[t], row0 = tile_row0[t], rows = tile_rows[t];
  const int h0 = blockIdx.y * hb;
  const int nh = min(hb, heads - h0);
  const int nq = rows * nh;
  const int p0 = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int qi = warp; qi < nq; qi += kWarps) {
    const act_t* src = q + static_cast<size_t>(row0 + qi / nh) * q_stride + (h0 + qi % nh) * dk;
    for (int d = lane; d < dk; d += 32) qs[qi * dk + d] = bw::to_f(src[d]);
  }
  float m[QW], l[QW], acc[QW][ACC];
#pragma unroll
  for (int j = 0; j < QW; ++j) {
    m[j] = -INFINITY, l[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[j][i] = 0.0f;
  }
  const int last = p0 + rows - 1;
  const int first = window > 0 ? max(0, p0 - window + 1) : 0;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  for (int k0 = first / kKeys * kKeys; k0 <= last; k0 += kKeys) {
    __syncthreads();
    load_keys(keys, ks, cache, bt, page, dk, k0, last, warp, lane);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < QW; ++j) {
      const int qi = warp + kWarps * j;
      if (qi >= nq) continue;
      const int pq = p0 + qi / nh;
      const int lo = window > 0 ? max(0, pq - window + 1) : 0;
      attend_tile<ACC>(keys, ks, qs + qi * dk, dk, rank, k0, lo, pq, scale, lane, m[j], l[j], acc[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < QW; ++j) {
    const int qi = warp + kWarps * j;
    if (qi >= nq) continue;
    act_t* dst = out + static_cast<size_t>(row0 + qi / nh) * o_stride + (h0 + qi % nh) * rank;
    const float inv = __fdiv_rn(1.0f, with_sink(l[j], m[j], sinks, h0 + qi % nh));
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int d = i * 32 + lane;
      if (d < rank) dst[d] = bw::from_f<act_t>(__fmul_rn(acc[j][i], inv));
    }
  }
}

// Steps of single rows: the keys of a row are cut into spans of `span` keys (a multiple of 32,
// at fixed absolute positions); a block takes one span of one row and up to kWarps heads, walks
// the span's tiles as above, and leaves (m, l, weighted sum) per head and span. The merge folds
// a query's spans in ascending order.
template <int ACC>
__global__ void __launch_bounds__(kThreads)
latent_attention_split_kernel(const act_t* __restrict__ q, int q_stride, const act_t* __restrict__ cache,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seq,
                              const int* __restrict__ pos, float* __restrict__ part, int spans, int span, int heads,
                              int rank, int rot_dim, int page, int window, float scale) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int dk = rank + rot_dim, ks = dk + 1;
  float* keys = sm;
  float* qs = sm + kKeys * ks;
  const int r = blockIdx.x, sp = blockIdx.y, h0 = blockIdx.z * kWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = h0 + warp;
  const int pq = pos[r];
  const int lo = window > 0 ? max(0, pq - window + 1) : 0;
  const int begin = max(sp * span, lo / kKeys * kKeys), end = min(pq, (sp + 1) * span - 1);
  float* rec = part + ((static_cast<size_t>(r) * heads + h) * spans + sp) * (rank + 2);
  if (begin > end) {  // nothing of this span is seen
    if (h < heads && lane == 0) rec[0] = -INFINITY, rec[1] = 0.0f;
    return;
  }
  if (h < heads) {
    const act_t* src = q + static_cast<size_t>(r) * q_stride + h * dk;
    for (int d = lane; d < dk; d += 32) qs[warp * dk + d] = bw::to_f(src[d]);
  }
  float m = -INFINITY, l = 0.0f, acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.0f;
  const int* bt = block_table + static_cast<size_t>(row_seq[r]) * max_blocks;
  for (int k0 = begin; k0 <= end; k0 += kKeys) {
    __syncthreads();
    load_keys(keys, ks, cache, bt, page, dk, k0, end, warp, lane);
    __syncthreads();
    if (h < heads) attend_tile<ACC>(keys, ks, qs + warp * dk, dk, rank, k0, lo, pq, scale, lane, m, l, acc);
  }
  if (h >= heads) return;
  if (lane == 0) rec[0] = m, rec[1] = l;
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int d = i * 32 + lane;
    if (d < rank) rec[2 + d] = acc[i];
  }
}

// One block per (row, head): folds the spans' records in ascending order.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part, const int* __restrict__ pos, int spans, int span,
                              int heads, int rank, act_t* out, int o_stride, const float* __restrict__ sinks) {
  bw::pdl_enter();
  const int r = blockIdx.x, h = blockIdx.y;
  const float* rec0 = part + (static_cast<size_t>(r) * heads + h) * spans * (rank + 2);
  const int used = min(spans, pos[r] / span + 1);
  float m = -INFINITY;
  for (int s = 0; s < used; ++s) m = fmaxf(m, rec0[static_cast<size_t>(s) * (rank + 2)]);
  float l = 0.0f;
  for (int s = 0; s < used; ++s) {
    const float* rec = rec0 + static_cast<size_t>(s) * (rank + 2);
    if (rec[0] != -INFINITY) l = __fmaf_rn(rec[1], expf(__fsub_rn(rec[0], m)), l);
  }
  const float inv = __fdiv_rn(1.0f, with_sink(l, m, sinks, h));
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float a = 0.0f;
    for (int s = 0; s < used; ++s) {
      const float* rec = rec0 + static_cast<size_t>(s) * (rank + 2);
      if (rec[0] != -INFINITY) a = __fmaf_rn(rec[2 + d], expf(__fsub_rn(rec[0], m)), a);
    }
    out[static_cast<size_t>(r) * o_stride + h * rank + d] = bw::from_f<act_t>(__fmul_rn(a, inv));
  }
}

#if BW_ACT_BF16
// ---------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16 serving precision). A block takes up to 64
// queries, (row, head) pairs of one query tile with the heads running fastest, and walks its
// keys in tiles of 32 at the fixed absolute positions, two tiles in flight (cp.async). Four
// warps own 16 queries each: scores S = Q K^T by mma.sync over rank + rot_dim (float32
// accumulators: the scores are 32-bit), scaling, mask, running maximum and sum in float32, and
// the weights enter the second product in two bfloat16 parts, p = hi + lo with lo = p - hi, so
// that what multiplies the latents carries 16 bits of the float32 weight and not 8. The latents
// of the tile (the first `rank` columns of the same shared-memory rows) are the second
// product's right operand. With CS = 2 a second set of four warps owns the other half of the
// latent columns (a warp's accumulators are 16 x NT * 8 floats); each set forms the scores of
// half of a tile's keys and both read the whole tile's scores back from shared memory.
// With `part` the block covers one span of keys and leaves (maximum, sum, unnormalised sum of
// latents) per query for the merge; else it writes the finished rows.
constexpr int kTcKeys = 32, kTcQueries = 64, kScoreRow = kTcKeys + 8;  // 40 floats: rows 8 apart fall on other banks

template <int NT, int CS>
__global__ void __launch_bounds__(128 * CS)
latent_attention_tc_kernel(const act_t* __restrict__ q, int q_stride, const act_t* __restrict__ cache,
                           const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tile_seq,
                           const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                           const int* __restrict__ seq_pos0, const int* __restrict__ seq_row0, act_t* out, int o_stride,
                           float* __restrict__ part, int spans, int span, int heads, int hb, int rank, int rot_dim,
                           int page, int window, float scale, const float* __restrict__ sinks) {
  bw::pdl_enter();
  extern __shared__ __align__(16) unsigned char raw[];
  const int dk = rank + rot_dim, rs = dk + 8;  // row stride in elements: an odd number of 16-byte pieces
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(raw);
  __nv_bfloat16* ks = qs + kTcQueries * rs;   // two tiles of kTcKeys rows
  float* ss = reinterpret_cast<float*>(ks + 2 * kTcKeys * rs);  // CS == 2: a tile's scores, [queries][kScoreRow]
  const int t = blockIdx.x, sp = blockIdx.z;
  const int seq = tile_seq[t], row0 = tile_row0[t], rows = tile_rows[t];
  const int h0 = blockIdx.y * hb;
  const int nh = min(hb, heads - h0);
  const int nq = rows * nh;
  const int p0 = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wq = warp & 3, cs = warp >> 2;
  const int threads = 128 * CS, pieces = dk >> 3;
  const int last = p0 + rows - 1;
  const int first = window > 0 ? max(0, p0 - window + 1) : 0;
  const int kbeg = max(sp * span, first / kTcKeys * kTcKeys), kend = min(last, (sp + 1) * span - 1);
  const int tiles = kbeg <= kend ? (kend - kbeg) / kTcKeys + 1 : 0;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;

  for (int idx = tid; idx < kTcQueries * pieces; idx += threads) {
    const int qi = idx / pieces, c = idx - qi * pieces;
    const bool valid = qi < nq;
    const act_t* src = valid ? q + static_cast<size_t>(row0 + qi / nh) * q_stride + (h0 + qi % nh) * dk + c * 8 : q;
    bw::copy16_async(bw::smem_addr(qs + qi * rs + c * 8), src, valid);
  }
  // a warp copies whole keys: the page is looked up once per key, the lanes share its 16-byte pieces
  auto load_keys_async = [&](int tile) {
    __nv_bfloat16* dst = ks + (tile & 1) * kTcKeys * rs;
    const int k0 = kbeg + tile * kTcKeys;
    for (int kk = warp; kk < kTcKeys; kk += 4 * CS) {
      const int kp = k0 + kk;
      const bool valid = kp <= kend;
      const act_t* src = valid ? cache + (static_cast<size_t>(bt[kp / page]) * page + kp % page) * dk : cache;
      for (int c = lane; c < pieces; c += 32) bw::copy16_async(bw::smem_addr(dst + kk * rs + c * 8), valid ? src + c * 8 : cache, valid);
    }
  };
  if (tiles > 0) load_keys_async(0);
  bw::copies_commit();

  // the two query rows of this thread's accumulator fragments
  const int qa = wq * 16 + (lane >> 2), qb = qa + 8;
  const int pa = qa < nq ? p0 + qa / nh : -1, pb = qb < nq ? p0 + qb / nh : -1;
  const int la = window > 0 ? max(0, pa - window + 1) : 0, lb = window > 0 ? max(0, pb - window + 1) : 0;
  float ma = -INFINITY, mb = -INFINITY, suma = 0.0f, sumb = 0.0f;
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

  for (int tile = 0; tile < tiles; ++tile) {
    if (tile + 1 < tiles) load_keys_async(tile + 1);
    bw::copies_commit();
    bw::copies_wait<1>();
    __syncthreads();
    const __nv_bfloat16* kt = ks + (tile & 1) * kTcKeys * rs;
    const int k0 = kbeg + tile * kTcKeys;
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
    // The fragments of step k + 1 are requested before the products of step k are issued, and
    // even and odd steps add into accumulators of their own (summed at the end), so that neither
    // the loads nor the chain of dependent products stand in the warp's way.
    const uint32_t q_at = bw::smem_addr(qs + (wq * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * rs + 8 * (lane >> 4));
    const uint32_t k_at = bw::smem_addr(kt + ((lane & 7) + 8 * (lane >> 4)) * rs + 8 * ((lane >> 3) & 1));
    if constexpr (CS == 1) {
      float odd[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) odd[j][0] = odd[j][1] = odd[j][2] = odd[j][3] = 0.0f;
      uint32_t a0[4], b00[4], b01[4], a1[4], b10[4], b11[4];
      int kk = 0;
      bw::ldsm4(a0, q_at), bw::ldsm4(b00, k_at), bw::ldsm4(b01, k_at + 16 * rs * 2);
      for (; kk + 16 < dk; kk += 32) {
        bw::ldsm4(a1, q_at + (kk + 16) * 2), bw::ldsm4(b10, k_at + (kk + 16) * 2), bw::ldsm4(b11, k_at + (16 * rs + kk + 16) * 2);
        bw::mma16816(sc[0], a0, b00[0], b00[1]), bw::mma16816(sc[1], a0, b00[2], b00[3]);
        bw::mma16816(sc[2], a0, b01[0], b01[1]), bw::mma16816(sc[3], a0, b01[2], b01[3]);
        if (kk + 32 < dk)
          bw::ldsm4(a0, q_at + (kk + 32) * 2), bw::ldsm4(b00, k_at + (kk + 32) * 2), bw::ldsm4(b01, k_at + (16 * rs + kk + 32) * 2);
        bw::mma16816(odd[0], a1, b10[0], b10[1]), bw::mma16816(odd[1], a1, b10[2], b10[3]);
        bw::mma16816(odd[2], a1, b11[0], b11[1]), bw::mma16816(odd[3], a1, b11[2], b11[3]);
      }
      if (kk < dk) {
        bw::mma16816(sc[0], a0, b00[0], b00[1]), bw::mma16816(sc[1], a0, b00[2], b00[3]);
        bw::mma16816(sc[2], a0, b01[0], b01[1]), bw::mma16816(sc[3], a0, b01[2], b01[3]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[j][e] += odd[j][e];
    } else {
      // each set of warps forms the scores of half of the tile's keys and hands them to the other
      // through shared memory (a score is the same chain either way)
      float half[2][4], odd[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) half[j][e] = odd[j][e] = 0.0f;
      const uint32_t kh_at = k_at + 16 * cs * rs * 2;
      uint32_t a0[4], b0[4], a1[4], b1[4];
      int kk = 0;
      bw::ldsm4(a0, q_at), bw::ldsm4(b0, kh_at);
      for (; kk + 16 < dk; kk += 32) {
        bw::ldsm4(a1, q_at + (kk + 16) * 2), bw::ldsm4(b1, kh_at + (kk + 16) * 2);
        bw::mma16816(half[0], a0, b0[0], b0[1]), bw::mma16816(half[1], a0, b0[2], b0[3]);
        if (kk + 32 < dk) bw::ldsm4(a0, q_at + (kk + 32) * 2), bw::ldsm4(b0, kh_at + (kk + 32) * 2);
        bw::mma16816(odd[0], a1, b1[0], b1[1]), bw::mma16816(odd[1], a1, b1[2], b1[3]);
      }
      if (kk < dk) bw::mma16816(half[0], a0, b0[0], b0[1]), bw::mma16816(half[1], a0, b0[2], b0[3]);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) half[j][e] += odd[j][e];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float* dst = ss + qa * kScoreRow + 16 * cs + 8 * j + 2 * (lane & 3);
        *reinterpret_cast<float2*>(dst) = make_float2(half[j][0], half[j][1]);
        *reinterpret_cast<float2*>(dst + 8 * kScoreRow) = make_float2(half[j][2], half[j][3]);
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float* src = ss + qa * kScoreRow + 8 * j + 2 * (lane & 3);
        const float2 u = *reinterpret_cast<const float2*>(src), v = *reinterpret_cast<const float2*>(src + 8 * kScoreRow);
        sc[j][0] = u.x, sc[j][1] = u.y, sc[j][2] = v.x, sc[j][3] = v.y;
      }
    }
    float ta = -INFINITY, tb = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = k0 + 8 * j + 2 * (lane & 3) + e;
        const bool in_span = kp <= kend;
        sc[j][e] = (in_span && kp <= pa && kp >= la) ? __fmul_rn(sc[j][e], scale) : -INFINITY;
        sc[j][2 + e] = (in_span && kp <= pb && kp >= lb) ? __fmul_rn(sc[j][2 + e], scale) : -INFINITY;
        ta = fmaxf(ta, sc[j][e]), tb = fmaxf(tb, sc[j][2 + e]);
      }
    ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 1)), ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 2));
    tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 1)), tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 2));
    const float na = fmaxf(ma, ta), nb = fmaxf(mb, tb);
    const float base_a = na == -INFINITY ? 0.0f : na, base_b = nb == -INFINITY ? 0.0f : nb;
    const float alpha_a = __expf(ma - base_a), alpha_b = __expf(mb - base_b);  // exp(-inf) = 0
    ma = na, mb = nb;
    float ra = 0.0f, rb = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sc[j][e] = __expf(sc[j][e] - base_a), sc[j][2 + e] = __expf(sc[j][2 + e] - base_b);
        ra += sc[j][e], rb += sc[j][2 + e];
      }
    suma = __fmaf_rn(suma, alpha_a, ra), sumb = __fmaf_rn(sumb, alpha_b, rb);
    // once a row's maximum stands, its factor is 1: most tiles rescale nothing
    if (__any_sync(0xffffffffu, alpha_a != 1.0f || alpha_b != 1.0f)) {
#pragma unroll
      for (int i = 0; i < NT; ++i) acc[i][0] *= alpha_a, acc[i][1] *= alpha_a, acc[i][2] *= alpha_b, acc[i][3] *= alpha_b;
    }
#pragma unroll
    for (int k2 = 0; k2 < 2; ++k2) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const float v0 = sc[2 * k2 + (f >> 1)][(f & 1) * 2], v1 = sc[2 * k2 + (f >> 1)][(f & 1) * 2 + 1];
        const __nv_bfloat16 h0b = __float2bfloat16_rn(v0), h1b = __float2bfloat16_rn(v1);
        hi[f] = bw::pack_bf16(v0, v1);
        lo[f] = bw::pack_bf16(v0 - __bfloat162float(h0b), v1 - __bfloat162float(h1b));
      }
      const uint32_t v_at = bw::smem_addr(kt + (k2 * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * rs + 8 * (lane >> 4));
#pragma unroll
      for (int n4 = 0; n4 < NT / 2; n4 += 4) {
        // four fragments of latents are requested, then their products follow, the high parts of
        // the weights first: no product waits for the one before it on the same accumulator
        uint32_t b[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int d0 = (cs * NT + 2 * (n4 + u)) * 8;
          if (d0 < rank) bw::ldsm4_trans(b[u], v_at + d0 * 2);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if ((cs * NT + 2 * (n4 + u)) * 8 < rank) {
            bw::mma16816(acc[2 * (n4 + u)], hi, b[u][0], b[u][1]);
            bw::mma16816(acc[2 * (n4 + u) + 1], hi, b[u][2], b[u][3]);
          }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if ((cs * NT + 2 * (n4 + u)) * 8 < rank) {
            bw::mma16816(acc[2 * (n4 + u)], lo, b[u][0], b[u][1]);
            bw::mma16816(acc[2 * (n4 + u) + 1], lo, b[u][2], b[u][3]);
          }
      }
    }
    __syncthreads();
  }
  bw::copies_wait<0>();
  suma += __shfl_xor_sync(0xffffffffu, suma, 1), suma += __shfl_xor_sync(0xffffffffu, suma, 2);
  sumb += __shfl_xor_sync(0xffffffffu, sumb, 1), sumb += __shfl_xor_sync(0xffffffffu, sumb, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int qi = half ? qb : qa;
    if (qi >= nq) continue;
    const int row = row0 + qi / nh, h = h0 + qi % nh;
    const float m = half ? mb : ma, l = half ? sumb : suma;
    if (part) {
      float* rec = part + ((static_cast<size_t>(row) * heads + h) * spans + sp) * (rank + 2);
      if (cs == 0 && (lane & 3) == 0) rec[0] = m, rec[1] = l;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int d = (cs * NT + i) * 8 + 2 * (lane & 3);
        if (d < rank) rec[2 + d] = acc[i][2 * half], rec[3 + d] = acc[i][2 * half + 1];
      }
    } else {
      const float inv = __fdiv_rn(1.0f, with_sink(l, m, sinks, h));
      act_t* dst = out + static_cast<size_t>(row) * o_stride + h * rank;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int d = (cs * NT + i) * 8 + 2 * (lane & 3);
        if (d < rank) *reinterpret_cast<uint32_t*>(dst + d) = bw::pack_bf16(acc[i][2 * half] * inv, acc[i][2 * half + 1] * inv);
      }
    }
  }
}

int g_force_plain_attention = 0;
#endif

size_t attention_smem(int rank, int rot_dim, int queries) {
  const int dk = rank + rot_dim;
  return (static_cast<size_t>(kKeys) * (dk + 1) + static_cast<size_t>(queries) * dk) * sizeof(float);
}

template <typename K>
int raise_smem(K kernel, size_t smem) {
  if (smem <= 48 * 1024) return 0;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    bw::set_error("latent attention: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return 0;
}

constexpr int kQueriesPerWarp = 4;

}  // namespace

BW_API int BW_FN(latent_store)(const float* d, int d_stride, const float* w, float eps, const int* pos,
                               const int* row_seq, const float* cos_t, const float* sin_t, int pairs,
                               const int* block_table, int max_blocks, act_t* cache, int n, int rank, int rot_dim,
                               int page, int half_layout, const float* q_w, int q_rank, act_t* q_out,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  if (half_layout && pairs == 0) half_layout = 0;
  if (q_out && (!q_w || q_rank <= 0)) {
    bw::set_error("latent_store: the queries' latent needs a weight and a size");
    return -1;
  }
  if (rank <= 0 || rot_dim < 0 || 2 * pairs > rot_dim || (pairs > 0 && !cos_t)) {
    bw::set_error("latent_store: rank %d, rotated part %d, %d pairs", rank, rot_dim, pairs);
    return -1;
  }
  bw::launch_pdl(latent_store_kernel, dim3(n), dim3(128), 0, stream, d, d_stride, w, eps, pos, row_seq, cos_t, sin_t,
                 pairs, block_table, max_blocks, cache, rank, rot_dim, page, half_layout, q_w, q_rank, q_out);
  return bw::launch_status();
}

BW_API int BW_FN(rotate_heads)(const act_t* q, int q_stride, int head_stride, int offset, act_t* out, int o_stride,
                               int out_head_stride, int out_offset, int n, int heads, int rot_dim, int pairs,
                               const int* pos, const float* cos_t, const float* sin_t, int half_layout,
                               cudaStream_t stream) {
  if (n <= 0 || heads <= 0 || rot_dim <= 0) return 0;
  if (half_layout && pairs == 0) half_layout = 0;
  if (2 * pairs > rot_dim || (pairs > 0 && !cos_t)) {
    bw::set_error("rotate_heads: %d heads, rotated part %d, %d pairs", heads, rot_dim, pairs);
    return -1;
  }
  bw::launch_pdl(rotate_heads_kernel, dim3(n), dim3(128), 0, stream, q, q_stride, head_stride, offset, out, o_stride,
                 out_head_stride, out_offset, heads, rot_dim, pairs, pos, cos_t, sin_t, half_layout);
  return bw::launch_status();
}

// Rows of one sequence that a query tile of this many heads holds (the tile height the caller
// prepares), and the heads a block takes.
BW_API int BW_FN(latent_attention_tile_rows)(int heads) {
  const int q = kWarps * kQueriesPerWarp;
  return heads >= q ? 1 : q / heads;
}

BW_API int BW_FN(latent_attention)(const act_t* q, int q_stride, const act_t* cache, const int* block_table,
                                   int max_blocks, const int* tile_seq, const int* tile_row0, const int* tile_rows,
                                   int tiles, const int* seq_pos0, const int* seq_row0, act_t* out, int o_stride,
                                   int heads, int rank, int rot_dim, int page, int window, float scale,
                                   const float* sinks, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  const int q_max = kWarps * kQueriesPerWarp;
  const int hb = heads < q_max ? heads : q_max;
  const size_t smem = attention_smem(rank, rot_dim, q_max);
  if (rank > 512 || smem > 200 * 1024) {
    bw::set_error("latent attention: latent size %d with rotated part %d is beyond the kernel (512, %zu bytes)", rank,
                  rot_dim, smem);
    return -1;
  }
  dim3 grid(tiles, (heads + hb - 1) / hb);
#define BW_LAUNCH(ACC)                                                                                              \
  {                                                                                                                 \
    auto kernel = latent_attention_kernel<ACC, kQueriesPerWarp>;                                                    \
    if (int rc = raise_smem(kernel, smem)) return rc;                                                               \
    bw::launch_pdl(kernel, grid, dim3(kThreads), smem, stream, q, q_stride, cache, block_table, max_blocks, tile_seq, \
                   tile_row0, tile_rows, seq_pos0, seq_row0, out, o_stride, heads, hb, rank, rot_dim, page, window, \
                   scale, sinks);                                                                                   \
  }
  if (rank <= 128) BW_LAUNCH(4) else if (rank <= 256) BW_LAUNCH(8) else BW_LAUNCH(16)
#undef BW_LAUNCH
  return bw::launch_status();
}

// The split over keys for steps of single rows. `max_keys` bounds pos + 1 over the step; the
// span is chosen from it and from the number of rows so that the step fills the machine, and is
// a multiple of 32. Scratch: n * heads * spans * (rank + 2) floats.
BW_API int BW_FN(latent_attention_spans)(int n, int heads, int max_keys, int* span_out) {
  const int head_blocks = (heads + kWarps - 1) / kWarps;
  int want = (2 * 148 + n * head_blocks - 1) / (n * head_blocks);  // spans per row for two blocks per SM
  if (want < 1) want = 1;
  int span = (max_keys + want - 1) / want;
  span = (span + 127) / 128 * 128;  // at least four tiles per block
  *span_out = span;
  return (max_keys + span - 1) / span;
}

BW_API int BW_FN(latent_attention_split)(const act_t* q, int q_stride, const act_t* cache, const int* block_table,
                                         int max_blocks, const int* row_seq, const int* pos, act_t* out, int o_stride,
                                         int n, int heads, int rank, int rot_dim, int page, int window, float scale,
                                         int max_keys, float* scratch, const float* sinks, cudaStream_t stream) {
  if (n <= 0) return 0;
  int span = 0;
  const int spans = BW_FN(latent_attention_spans)(n, heads, max_keys, &span);
  const size_t smem = attention_smem(rank, rot_dim, kWarps);
  if (rank > 512 || smem > 200 * 1024 || spans > 65535) {
    bw::set_error("latent attention: latent size %d with rotated part %d is beyond the kernel", rank, rot_dim);
    return -1;
  }
  dim3 grid(n, spans, (heads + kWarps - 1) / kWarps);
#define BW_LAUNCH(ACC)                                                                                               \
  {                                                                                                                  \
    auto kernel = latent_attention_split_kernel<ACC>;                                                                \
    if (int rc = raise_smem(kernel, smem)) return rc;                                                                \
    bw::launch_pdl(kernel, grid, dim3(kThreads), smem, stream, q, q_stride, cache, block_table, max_blocks, row_seq,  \
                   pos, scratch, spans, span, heads, rank, rot_dim, page, window, scale);                            \
  }
  if (rank <= 128) BW_LAUNCH(4) else if (rank <= 256) BW_LAUNCH(8) else BW_LAUNCH(16)
#undef BW_LAUNCH
  if (int rc = bw::launch_status()) return rc;
  bw::launch_pdl(latent_attention_merge_kernel, dim3(n, heads), dim3(128), 0, stream, scratch, pos, spans, span, heads,
                 rank, out, o_stride, sinks);
  return bw::launch_status();
}

#if BW_ACT_BF16
// Tests: 1 keeps attention on the plain kernels also where the tensor-core kernel would take
// the shape. Returns the setting before.
BW_API int BW_FN(latent_attention_force_plain)(int on) {
  const int was = g_force_plain_attention;
  g_force_plain_attention = on;
  return was;
}

// Rows of one sequence per query tile for the tensor-core kernel, 0 where it does not take the
// shape (the latent size a multiple of 8 up to 512, rank + rot_dim a multiple of 16, rows that
// start on 16 bytes).
BW_API int BW_FN(latent_attention_tc_tile_rows)(int heads, int rank, int rot_dim, int q_stride) {
  const int dk = rank + rot_dim;
  const size_t smem = static_cast<size_t>(kTcQueries + 2 * kTcKeys) * (dk + 8) * 2 + kTcQueries * kScoreRow * 4;
  if (g_force_plain_attention || rank % 8 || dk % 16 || rank > 512 || q_stride % 8 || smem > 200 * 1024) return 0;
  return heads >= kTcQueries ? 1 : kTcQueries / heads;
}

// Spans for steps of single rows: enough blocks for two per SM, spans of whole key tiles.
BW_API int BW_FN(latent_attention_tc_spans)(int tiles, int heads, int max_keys, int* span_out) {
  const int hb = heads < kTcQueries ? heads : kTcQueries;
  const int blocks = tiles * ((heads + hb - 1) / hb);
  int want = (2 * 148 + blocks - 1) / blocks;
  if (want < 1) want = 1;
  int span = (max_keys + want - 1) / want;
  span = (span + 127) / 128 * 128;
  *span_out = span;
  return (max_keys + span - 1) / span;
}

// `scratch` null: query tiles of any height, finished rows. Else every tile is a single row, the
// keys are split into spans (latent_attention_tc_spans) and the merge follows.
BW_API int BW_FN(latent_attention_tc)(const act_t* q, int q_stride, const act_t* cache, const int* block_table,
                                      int max_blocks, const int* tile_seq, const int* tile_row0, const int* tile_rows,
                                      int tiles, const int* seq_pos0, const int* seq_row0, const int* pos, act_t* out,
                                      int o_stride, int n, int heads, int rank, int rot_dim, int page, int window,
                                      float scale, int max_keys, float* scratch, const float* sinks, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (!BW_FN(latent_attention_tc_tile_rows)(heads, rank, rot_dim, q_stride) || o_stride % 2) {
    bw::set_error("latent attention: the tensor-core kernel does not take rank %d with rotated part %d", rank, rot_dim);
    return -1;
  }
  const int dk = rank + rot_dim;
  const int hb = heads < kTcQueries ? heads : kTcQueries;
  const size_t smem = static_cast<size_t>(kTcQueries + 2 * kTcKeys) * (dk + 8) * 2 + kTcQueries * kScoreRow * 4;
  int spans = 1, span = 1 << 30;
  if (scratch) spans = BW_FN(latent_attention_tc_spans)(tiles, heads, max_keys, &span);
  dim3 grid(tiles, (heads + hb - 1) / hb, spans);
#define BW_LAUNCH(NT, CS)                                                                                          \
  {                                                                                                                \
    auto kernel = latent_attention_tc_kernel<NT, CS>;                                                              \
    if (int rc = raise_smem(kernel, smem)) return rc;                                                              \
    bw::launch_pdl(kernel, grid, dim3(128 * CS), smem, stream, q, q_stride, cache, block_table, max_blocks,        \
                   tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out, o_stride, scratch, spans, span, heads, \
                   hb, rank, rot_dim, page, window, scale, sinks);                                                 \
  }
  if (rank <= 128) BW_LAUNCH(16, 1) else if (rank <= 256) BW_LAUNCH(32, 1) else BW_LAUNCH(32, 2)
#undef BW_LAUNCH
  if (int rc = bw::launch_status()) return rc;
  if (scratch) {
    bw::launch_pdl(latent_attention_merge_kernel, dim3(n, heads), dim3(128), 0, stream, scratch, pos, spans, span, heads,
                   rank, out, o_stride, sinks);
    return bw::launch_status();
  }
  return 0;
}
#endif
