// A feed-forward of many small experts of which a row uses a few, and products per group.
//
//  * route: from a row's router logits (float32) to its experts and their weights. Scores are
//    sigmoid(z); a correction per expert is added for the choice only; the experts form equal
//    groups of neighbours, a group counts as the sum of its two largest choice scores, and only
//    the experts of the best groups can be chosen; the weights are the chosen experts' scores
//    times a constant. `softmax_top`: the choice is by the logits themselves (plus the correction), and
//    the weights are the softmax over the chosen logits only.
//  * group_rows: (row, choice) pairs listed expert by expert, with the tiles of the grouped
//    product that follows.
//  * grouped_linear: out[i] = x[source(i)] W_g^T for the list entries i of every group g, W
//    stored [groups, n, k]. With a list the groups are the experts (rows of unequal number);
//    without, every group takes every row and reads and writes its own columns (one product per
//    head). An output is one chain over k in ascending order, whatever tile it sits in: fused
//    multiply-adds on the CUDA cores, or on the serving precision tensor-core steps of 16.
//  * gather_rows: the rows of a list made contiguous, for the tcgen05 product over long lists
//    (bf16_gemm_tc.cu), which fetches tiles of consecutive rows.
//  * glu_clamped: y = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, +-limit).
//  * combine: x += d + sum_j weight_j * y[place of (row, j)], the sum in the order of choice.
#include "bw_act.cuh"
#include "bw_mma.cuh"

#include <math.h>

namespace {

// ---------------------------------------------------------------------------------------
// One warp per row. Shared memory per warp: scores s[E] (a taken expert's is set to -1), choice
// scores c[E] (-inf for the experts of groups that do not stay), group scores [groups].
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ z, const float* __restrict__ correction, int n, int experts, int groups,
             int keep, int top, float weight_scale, int softmax_top, int* __restrict__ chosen,
             float* __restrict__ weights) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= n) return;
  float* s = sm + static_cast<size_t>(warp) * (2 * experts + groups);
  float* c = s + experts;
  float* gs = c + experts;
  const float* zr = z + static_cast<size_t>(r) * experts;
  for (int e = lane; e < experts; e += 32) {
    const float v = softmax_top ? zr[e] : __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-zr[e])));
    s[e] = softmax_top ? 0.0f : v;  // (only its sign is used then: negative once taken)
    c[e] = correction ? __fadd_rn(v, correction[e]) : v;
  }
  __syncwarp();
  const int per = experts / groups;
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;  // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = c[e];
        if (v > a) b = a, a = v;
        else if (v > b) b = v;
      }
      gs[g] = per > 1 ? __fadd_rn(a, b) : a;
    }
    __syncwarp();
    // the groups that stay are taken out of gs one by one (marked +inf); the rest lose their experts
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || at == 0x7fffffff)) best = v, at = g;
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) best = ob, at = oa;
      }
      if (lane == 0 && at != 0x7fffffff) gs[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / per] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  // a taken expert is marked by a negative score (scores lie in (0, 1)) once its weight is read
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c[e];
      if (s[e] >= 0.0f && (at == 0x7fffffff || v > best)) best = v, at = e;
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) best = ob, at = oa;
    }
    if (lane == 0) {
      chosen[static_cast<size_t>(r) * top + k] = at;
      weights[static_cast<size_t>(r) * top + k] = softmax_top ? zr[at] : __fmul_rn(s[at], weight_scale);
      s[at] = -1.0f;  // taken
    }
    __syncwarp();
  }
  if (softmax_top && lane == 0) {
    // the softmax over the chosen logits, in the order of choice (the first is the largest)
    float* wr = weights + static_cast<size_t>(r) * top;
    float m = wr[0];
    for (int k = 1; k < top; ++k) m = fmaxf(m, wr[k]);
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      const float e = expf(__fsub_rn(wr[k], m));
      wr[k] = e;
      sum = __fadd_rn(sum, e);
    }
    for (int k = 0; k < top; ++k) wr[k] = __fmul_rn(__fdiv_rn(wr[k], sum), weight_scale);
  }
}

// ---------------------------------------------------------------------------------------
// pairs = n * top entries of `chosen`. Every block counts the experts' pairs for itself (shared-memory
// atomics; the counts do not depend on their order); the placing is shared between the blocks. Outputs: group_off[E + 1] (where each
// expert's list begins), tile_prefix[2][E + 1] (tiles of `tile_rows` list entries before each
// expert, then tiles of twice as many), order[pairs] (the pairs expert by expert, ascending inside an expert) and
// place[pairs] (where a pair stands in that order).
__global__ void __launch_bounds__(1024)
group_rows_kernel(const int* __restrict__ chosen, int pairs, int experts, int tile_rows, int* __restrict__ group_off,
                  int* __restrict__ tile_prefix, int* __restrict__ order, int* __restrict__ place) {
  bw::pdl_enter();
  extern __shared__ int cnt[];  // [experts + 1]
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[chosen[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool writes = blockIdx.x == 0;  // every block counts, the first one writes the lists
    int rows = 0, tiles = 0, big = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = cnt[e];
      if (writes) group_off[e] = rows, tile_prefix[e] = tiles, tile_prefix[experts + 1 + e] = big;
      cnt[e] = rows;
      rows += c, tiles += (c + tile_rows - 1) / tile_rows, big += (c + 2 * tile_rows - 1) / (2 * tile_rows);
    }
    if (writes) group_off[experts] = rows, tile_prefix[experts] = tiles, tile_prefix[2 * experts + 1] = big;
  }
  __syncthreads();
  // a warp places the pairs of one expert; the experts are dealt to the warps of all blocks
  const int lane = threadIdx.x & 31, warps = (blockDim.x >> 5) * gridDim.x;
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (int e = warp; e < experts; e += warps) {
    int at = cnt[e];
    for (int p0 = 0; p0 < pairs; p0 += 256) {  // eight loads in flight: the walk is a chain of memory round trips
      int who[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int p = p0 + 32 * j + lane;
        who[j] = p < pairs ? chosen[p] : -1;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int p = p0 + 32 * j + lane;
        const bool mine = who[j] == e;
        const unsigned mask = __ballot_sync(0xffffffffu, mine);
        if (mine) {
          const int i = at + __popc(mask & ((1u << lane) - 1u));
          order[i] = p, place[p] = i;
        }
        at += __popc(mask);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// The grouped product: tiles of 64 list entries x 64 outputs, k in steps of 16, 256 threads with
// 4 x 4 outputs each.
constexpr int kTile = 64, kStep = 16;

template <typename OutT>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const act_t* __restrict__ x, int x_stride, int x_group_cols, const int* __restrict__ order,
                      int order_div, const act_t* __restrict__ w, OutT* out, int o_stride, int o_group_cols,
                      const int* __restrict__ group_off, const int* __restrict__ tile_prefix, int uniform_rows,
                      int groups, int n, int k) {
  bw::pdl_enter();
  __shared__ float xs[kStep][kTile + 1];
  __shared__ float ws[kStep][kTile + 1];
  __shared__ int s_group;
  int g, i0, i_end;
  if (group_off) {
    if (threadIdx.x == 0) {
      int found = -1;
      const int t = blockIdx.x;
      if (t < tile_prefix[groups]) {
        int lo = 0, hi = groups - 1;  // the last group whose first tile is at or before t and that has tiles
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (tile_prefix[mid] <= t) lo = mid; else hi = mid - 1;
        }
        found = lo;
      }
      s_group = found;
    }
    __syncthreads();
    g = s_group;
    if (g < 0) return;
    i0 = group_off[g] + (blockIdx.x - tile_prefix[g]) * kTile;
    i_end = group_off[g + 1];
  } else {
    const int tiles = (uniform_rows + kTile - 1) / kTile;
    g = blockIdx.x / tiles;
    i0 = (blockIdx.x - g * tiles) * kTile;
    i_end = uniform_rows;
  }
  const int j0 = blockIdx.y * kTile;
  const act_t* wg = w + static_cast<size_t>(g) * n * k;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // outputs (ty * 4 + a, tx * 4 + b)
  // what this thread loads each step: entry (threadIdx.x / 16) + 16 q of the tile, k index threadIdx.x % 16
  const int lk = threadIdx.x & 15, lr = threadIdx.x >> 4;
  const act_t* xrow[4];
  const act_t* wrow[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int i = i0 + lr + 16 * q;
    xrow[q] = nullptr;
    if (i < i_end) {
      const int src = order ? order[i] / order_div : i;
      xrow[q] = x + static_cast<size_t>(src) * x_stride + (group_off ? 0 : g * x_group_cols);
    }
    const int j = j0 + lr + 16 * q;
    wrow[q] = j < n ? wg + static_cast<size_t>(j) * k : nullptr;
  }
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
  for (int k0 = 0; k0 < k; k0 += kStep) {
    const int kk = k0 + lk;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      xs[lk][lr + 16 * q] = (xrow[q] && kk < k) ? bw::to_f(xrow[q][kk]) : 0.0f;
      ws[lk][lr + 16 * q] = (wrow[q] && kk < k) ? bw::to_f(wrow[q][kk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < kStep; ++s) {
      float xv[4], wv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) xv[a] = xs[s][ty * 4 + a], wv[a] = ws[s][tx * 4 + a];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = __fmaf_rn(xv[a], wv[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = i0 + ty * 4 + a;
    if (i >= i_end) continue;
    OutT* orow = out + static_cast<size_t>(i) * o_stride + (group_off ? 0 : g * o_group_cols);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int j = j0 + tx * 4 + b;
      if (j < n) orow[j] = bw::from_f<OutT>(acc[a][b]);
    }
  }
}

#if BW_ACT_BF16
// The same product on the tensor cores (bfloat16 in, float32 accumulators that walk k in
// ascending steps of 16): tiles of BM list entries x BN outputs by WM x WN warps, k in slices of
// 32 through a ring of cp.async stages. 64 x 64 by four warps for short lists (decode steps), 128 x
// 128 by eight warps where the lists are long. For rows that start on 16 bytes (k, the row
// strides and the groups' column offsets multiples of 8).
constexpr int kMmaK = 32, kMmaRow = kMmaK + 8;  // 80-byte rows: ldmatrix without bank conflicts

template <typename OutT, int BM, int BN, int WM, int WN, int STAGES>
__global__ void __launch_bounds__(WM * WN * 32)
grouped_linear_mma_kernel(const act_t* __restrict__ x, int x_stride, int x_group_cols, const int* __restrict__ order,
                          int order_div, const act_t* __restrict__ w, OutT* out, int o_stride, int o_group_cols,
                          const int* __restrict__ group_off, const int* __restrict__ tile_prefix, int uniform_rows,
                          int groups, int n, int k) {
  bw::pdl_enter();
  constexpr int THREADS = WM * WN * 32;
  constexpr int TM = BM / WM, TN = BN / WN, MI = TM / 16, NI = TN / 8;
  constexpr int XQ = BM * 4 / THREADS, WQ = BN * 4 / THREADS;  // 16-byte pieces a thread copies per slice
  static_assert(NI % 2 == 0 && XQ >= 1 && WQ >= 1, "tile shape");
  extern __shared__ __align__(16) unsigned char raw[];
  typedef __nv_bfloat16 (*Tile)[kMmaRow];
  __nv_bfloat16* xs_base = reinterpret_cast<__nv_bfloat16*>(raw);
  __nv_bfloat16* ws_base = xs_base + STAGES * BM * kMmaRow;
  __shared__ int s_group;
  int g, i0, i_end;
  if (group_off) {
    if (threadIdx.x == 0) {
      int found = -1;
      const int t = blockIdx.x;
      if (t < tile_prefix[groups]) {
        int lo = 0, hi = groups - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (tile_prefix[mid] <= t) lo = mid; else hi = mid - 1;
        }
        found = lo;
      }
      s_group = found;
    }
    __syncthreads();
    g = s_group;
    if (g < 0) return;
    i0 = group_off[g] + (blockIdx.x - tile_prefix[g]) * BM;
    i_end = group_off[g + 1];
  } else {
    const int tiles = (uniform_rows + BM - 1) / BM;
    g = blockIdx.x / tiles;
    i0 = (blockIdx.x - g * tiles) * BM;
    i_end = uniform_rows;
  }
  const int j0 = blockIdx.y * BN;
  const act_t* wg = w + static_cast<size_t>(g) * n * k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp / WN) * TM, wn = (warp % WN) * TN;
  // a thread copies piece (tid % 4) of rows tid / 4 + (THREADS / 4) q of both tiles
  const int piece = tid & 3, lr = tid >> 2;
  const act_t* xrow[XQ];
  const act_t* wrow[WQ];
#pragma unroll
  for (int q = 0; q < XQ; ++q) {
    const int i = i0 + lr + (THREADS / 4) * q;
    xrow[q] = nullptr;
    if (i < i_end) {
      const int src = order ? order[i] / order_div : i;
      xrow[q] = x + static_cast<size_t>(src) * x_stride + (group_off ? 0 : g * x_group_cols);
    }
  }
#pragma unroll
  for (int q = 0; q < WQ; ++q) {
    const int j = j0 + lr + (THREADS / 4) * q;
    wrow[q] = j < n ? wg + static_cast<size_t>(j) * k : nullptr;
  }
  const int slices = (k + kMmaK - 1) / kMmaK;
  auto load = [&](int slice) {
    const int st = slice % STAGES, kk = slice * kMmaK + piece * 8;
    Tile xs = reinterpret_cast<Tile>(xs_base + st * BM * kMmaRow);
    Tile ws = reinterpret_cast<Tile>(ws_base + st * BN * kMmaRow);
#pragma unroll
    for (int q = 0; q < XQ; ++q) {
      const bool v = xrow[q] && kk < k;
      bw::copy16_async(bw::smem_addr(&xs[lr + (THREADS / 4) * q][piece * 8]), v ? xrow[q] + kk : x, v);
    }
#pragma unroll
    for (int q = 0; q < WQ; ++q) {
      const bool v = wrow[q] && kk < k;
      bw::copy16_async(bw::smem_addr(&ws[lr + (THREADS / 4) * q][piece * 8]), v ? wrow[q] + kk : w, v);
    }
  };
  float acc[MI][NI][4];
#pragma unroll
  for (int a = 0; a < MI; ++a)
#pragma unroll
    for (int b = 0; b < NI; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.0f;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < slices) load(s);
    bw::copies_commit();
  }
  for (int slice = 0; slice < slices; ++slice) {
    bw::copies_wait<STAGES - 2>();
    __syncthreads();
    if (slice + STAGES - 1 < slices) load(slice + STAGES - 1);
    bw::copies_commit();
    const int st = slice % STAGES;
    Tile xs = reinterpret_cast<Tile>(xs_base + st * BM * kMmaRow);
    Tile ws = reinterpret_cast<Tile>(ws_base + st * BN * kMmaRow);
#pragma unroll
    for (int ks = 0; ks < kMmaK / 16; ++ks) {
      uint32_t a[MI][4], b[NI / 2][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        bw::ldsm4(a[mi], bw::smem_addr(&xs[wm + mi * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][ks * 16 + 8 * (lane >> 4)]));
#pragma unroll
      for (int np = 0; np < NI / 2; ++np)
        bw::ldsm4(b[np], bw::smem_addr(&ws[wn + np * 16 + (lane & 7) + 8 * (lane >> 4)][ks * 16 + 8 * ((lane >> 3) & 1)]));
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni) bw::mma16816(acc[mi][ni], a[mi], b[ni >> 1][(ni & 1) * 2], b[ni >> 1][(ni & 1) * 2 + 1]);
    }
  }
  bw::copies_wait<0>();
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = i0 + wm + mi * 16 + (lane >> 2) + 8 * half;
      if (i >= i_end) continue;
      OutT* orow = out + static_cast<size_t>(i) * o_stride + (group_off ? 0 : g * o_group_cols);
#pragma unroll
      for (int ni = 0; ni < NI; ++ni) {
        const int j = j0 + wn + ni * 8 + 2 * (lane & 3);
        if (j < n) orow[j] = bw::from_f<OutT>(acc[mi][ni][2 * half]);
        if (j + 1 < n) orow[j + 1] = bw::from_f<OutT>(acc[mi][ni][2 * half + 1]);
      }
    }
}

constexpr int kBigTile = 128;

template <typename OutT, int BM, int BN, int WM, int WN, int STAGES>
int launch_grouped_mma(dim3 grid, cudaStream_t stream, const act_t* x, int x_stride, int x_group_cols, const int* order,
                       int order_div, const act_t* w, OutT* out, int o_stride, int o_group_cols, const int* group_off,
                       const int* tile_prefix, int rows, int groups, int n, int k) {
  auto kernel = grouped_linear_mma_kernel<OutT, BM, BN, WM, WN, STAGES>;
  constexpr size_t smem = static_cast<size_t>(STAGES) * (BM + BN) * kMmaRow * sizeof(__nv_bfloat16);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("grouped_linear: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    raised = true;
  }
  bw::launch_pdl(kernel, grid, dim3(WM * WN * 32), smem, stream, x, x_stride, x_group_cols, order, order_div, w, out,
                 o_stride, o_group_cols, group_off, tile_prefix, rows, groups, n, k);
  return bw::launch_status();
}
#endif

// out[i] = x[order[i] / order_div]: the rows of a list made contiguous (16 bytes per thread where
// the rows allow it), for products that fetch their operands as tiles of consecutive rows.
__global__ void gather_rows_kernel(const act_t* __restrict__ x, const int* __restrict__ order, int order_div,
                                   act_t* __restrict__ out, int k, int vec) {
  bw::pdl_enter();
  const int i = blockIdx.x;
  const act_t* src = x + static_cast<size_t>(order[i] / order_div) * k;
  act_t* dst = out + static_cast<size_t>(i) * k;
  if (vec) {
    constexpr int per = 16 / sizeof(act_t);
    for (int c = threadIdx.x; c < k / per; c += blockDim.x)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else {
    for (int c = threadIdx.x; c < k; c += blockDim.x) dst[c] = src[c];
  }
}

// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float glu_one(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__fmul_rn(alpha, g))));
  return __fmul_rn(__fmul_rn(g, sig), __fadd_rn(u, 1.0f));
}

// Grid (row, block of columns). VEC: a thread takes 16 bytes of gate and of up (the inner size a
// multiple of 16 bytes' worth and the buffers aligned), else one column.
template <bool VEC>
__global__ void glu_clamped_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inter, float limit,
                                   float alpha) {
  bw::pdl_enter();
  constexpr int per = VEC ? 16 / static_cast<int>(sizeof(act_t)) : 1;
  const int r = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * per;
  if (c >= inter) return;
  const act_t* row = gate_up + static_cast<size_t>(r) * 2 * inter;
  act_t* dst = out + static_cast<size_t>(r) * inter + c;
  if (VEC) {
    const uint4 gv = *reinterpret_cast<const uint4*>(row + c), uv = *reinterpret_cast<const uint4*>(row + inter + c);
    const act_t* g = reinterpret_cast<const act_t*>(&gv);
    const act_t* u = reinterpret_cast<const act_t*>(&uv);
    __align__(16) act_t o[per];
#pragma unroll
    for (int e = 0; e < per; ++e) o[e] = bw::from_f<act_t>(glu_one(bw::to_f(g[e]), bw::to_f(u[e]), limit, alpha));
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
  } else {
    dst[0] = bw::from_f<act_t>(glu_one(bw::to_f(row[c]), bw::to_f(row[inter + c]), limit, alpha));
  }
}

// x[r] += d[r] + sum_j weights[r][j] * y[place[r * top + j]]; d may be null. With `scale` (one factor per
// column) what is added is multiplied by it first. VEC: four columns per thread (the width a multiple of 4).
template <bool VEC>
__global__ void combine_kernel(float* x, const float* __restrict__ d, const float* __restrict__ y,
                               const int* __restrict__ place, const float* __restrict__ weights, int top, int width,
                               const float* __restrict__ scale) {
  bw::pdl_enter();
  constexpr int per = VEC ? 4 : 1;
  const int r = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * per;
  if (c >= width) return;
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int j = 0; j < top; ++j) {
    const size_t p = static_cast<size_t>(r) * top + j;
    const float wj = weights[p];
    const float* yr = y + static_cast<size_t>(place[p]) * width + c;
    if constexpr (VEC) {
      const float4 v = *reinterpret_cast<const float4*>(yr);
      s[0] = __fmaf_rn(wj, v.x, s[0]), s[1] = __fmaf_rn(wj, v.y, s[1]);
      s[2] = __fmaf_rn(wj, v.z, s[2]), s[3] = __fmaf_rn(wj, v.w, s[3]);
    } else {
      s[0] = __fmaf_rn(wj, yr[0], s[0]);
    }
  }
  const size_t o = static_cast<size_t>(r) * width + c;
#pragma unroll
  for (int e = 0; e < per; ++e) {
    float v = s[e];
    if (d) v = __fadd_rn(d[o + e], v);
    x[o + e] = scale ? __fmaf_rn(scale[c + e], v, x[o + e]) : __fadd_rn(x[o + e], v);
  }
}

}  // namespace

BW_API int BW_FN(route)(const float* z, const float* correction, int n, int experts, int groups, int keep, int top,
                        float weight_scale, int softmax_top, int* chosen, float* weights, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (experts <= 0 || groups <= 0 || experts % groups || keep <= 0 || keep > groups || top <= 0 ||
      top > keep * (experts / groups)) {
    bw::set_error("route: %d experts in %d groups of which %d stay cannot give %d choices", experts, groups, keep, top);
    return -1;
  }
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * (2 * experts + groups) * sizeof(float);
  if (smem > 48 * 1024) {
    bw::set_error("route: %d experts are beyond the kernel", experts);
    return -1;
  }
  bw::launch_pdl(route_kernel, dim3((n + warps - 1) / warps), dim3(warps * 32), smem, stream, z, correction, n, experts,
                 groups, keep, top, weight_scale, softmax_top, chosen, weights);
  return bw::launch_status();
}

BW_API int BW_FN(grouped_tile_rows)() { return kTile; }

// Tests: 1 keeps every grouped product on the plain kernel (one chain of fused multiply-adds per
// output) also where the tensor-core kernel would take it. Returns the setting before.
static int g_force_plain = 0;
BW_API int BW_FN(grouped_force_plain)(int on) {
  const int was = g_force_plain;
  g_force_plain = on;
  return was;
}

BW_API int BW_FN(group_rows)(const int* chosen, int pairs, int experts, int* group_off, int* tile_prefix, int* order,
                             int* place, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (experts <= 0 || experts > 8192) {
    bw::set_error("group_rows: %d experts", experts);
    return -1;
  }
  // one block for short lists; for long ones a block per 8 experts (a warp walks all pairs once per expert)
  const int blocks = pairs < 2048 ? 1 : (experts + 7) / 8;
  const int threads = blocks == 1 ? 1024 : 256;
  bw::launch_pdl(group_rows_kernel, dim3(blocks), dim3(threads), static_cast<size_t>(experts + 1) * sizeof(int), stream,
                 chosen, pairs, experts, kTile, group_off, tile_prefix, order, place);
  return bw::launch_status();
}

// With a list (group_off, tile_prefix, order from group_rows; `rows` = its length): entry i of
// group g reads x[order[i] / order_div] (order null: x[i]) and writes out[i]. Without (group_off
// null): every group takes rows 0 .. rows-1, reads columns g * x_group_cols .. and writes columns
// g * o_group_cols ...
BW_API int BW_FN(grouped_linear)(const act_t* x, int x_stride, int x_group_cols, const int* order, int order_div,
                                 const act_t* w, void* out, int out_is_f32, int o_stride, int o_group_cols,
                                 const int* group_off, const int* tile_prefix, int rows, int groups, int n, int k,
                                 cudaStream_t stream) {
  if (rows <= 0 || groups <= 0 || n <= 0) return 0;
  if (k <= 0 || order_div <= 0) {
    bw::set_error("grouped_linear: inner size %d", k);
    return -1;
  }
  const long long tiles = group_off ? (rows + kTile - 1) / kTile + groups
                                    : static_cast<long long>(groups) * ((rows + kTile - 1) / kTile);
  dim3 grid(static_cast<unsigned>(tiles), (n + kTile - 1) / kTile);
  if (tiles > 0x7fffffffLL || grid.y > 65535u) {
    bw::set_error("grouped_linear: %lld tiles exceed the grid", tiles);
    return -1;
  }
#if BW_ACT_BF16
  const bool aligned = k % 8 == 0 && x_stride % 8 == 0 && x_group_cols % 8 == 0 &&
                       reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
  if (aligned && !g_force_plain) {
    // long lists (on average a big tile's worth of rows per group) take tiles of 128 x 128
    const bool big = static_cast<long long>(rows) >= (group_off ? static_cast<long long>(kBigTile) * groups : kBigTile) && n >= kBigTile;
    if (big) {
      const long long bt = group_off ? (rows + kBigTile - 1) / kBigTile + groups
                                     : static_cast<long long>(groups) * ((rows + kBigTile - 1) / kBigTile);
      dim3 bgrid(static_cast<unsigned>(bt), (n + kBigTile - 1) / kBigTile);
      const int* prefix = tile_prefix ? tile_prefix + groups + 1 : nullptr;
      if (out_is_f32)
        return launch_grouped_mma<float, 128, 128, 2, 4, 4>(bgrid, stream, x, x_stride, x_group_cols, order, order_div, w,
                                                            static_cast<float*>(out), o_stride, o_group_cols, group_off,
                                                            prefix, rows, groups, n, k);
      return launch_grouped_mma<act_t, 128, 128, 2, 4, 4>(bgrid, stream, x, x_stride, x_group_cols, order, order_div, w,
                                                          static_cast<act_t*>(out), o_stride, o_group_cols, group_off,
                                                          prefix, rows, groups, n, k);
    }
    if (out_is_f32)
      return launch_grouped_mma<float, 64, 64, 2, 2, 3>(grid, stream, x, x_stride, x_group_cols, order, order_div, w,
                                                        static_cast<float*>(out), o_stride, o_group_cols, group_off,
                                                        tile_prefix, rows, groups, n, k);
    return launch_grouped_mma<act_t, 64, 64, 2, 2, 3>(grid, stream, x, x_stride, x_group_cols, order, order_div, w,
                                                      static_cast<act_t*>(out), o_stride, o_group_cols, group_off,
                                                      tile_prefix, rows, groups, n, k);
  }
#endif
  if (out_is_f32)
    bw::launch_pdl(grouped_linear_kernel<float>, grid, dim3(256), 0, stream, x, x_stride, x_group_cols, order, order_div,
                   w, static_cast<float*>(out), o_stride, o_group_cols, group_off, tile_prefix, rows, groups, n, k);
  else
    bw::launch_pdl(grouped_linear_kernel<act_t>, grid, dim3(256), 0, stream, x, x_stride, x_group_cols, order, order_div,
                   w, static_cast<act_t*>(out), o_stride, o_group_cols, group_off, tile_prefix, rows, groups, n, k);
  return bw::launch_status();
}

BW_API int BW_FN(gather_rows)(const act_t* x, const int* order, int order_div, act_t* out, int rows, int k,
                              cudaStream_t stream) {
  if (rows <= 0 || k <= 0) return 0;
  const int per = 16 / static_cast<int>(sizeof(act_t));
  const int vec = k % per == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  bw::launch_pdl(gather_rows_kernel, dim3(rows), dim3(128), 0, stream, x, order, order_div, out, k, vec);
  return bw::launch_status();
}

BW_API int BW_FN(glu_clamped)(const act_t* gate_up, act_t* out, int n, int inter, float limit, float alpha,
                              cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  const int per = 16 / static_cast<int>(sizeof(act_t));
  if (inter % per == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0)
    bw::launch_pdl(glu_clamped_kernel<true>, dim3(n, (inter / per + 127) / 128), dim3(128), 0, stream, gate_up, out, inter,
                   limit, alpha);
  else
    bw::launch_pdl(glu_clamped_kernel<false>, dim3(n, (inter + 255) / 256), dim3(256), 0, stream, gate_up, out, inter, limit,
                   alpha);
  return bw::launch_status();
}

BW_API int BW_FN(combine)(float* x, const float* d, const float* y, const int* place, const float* weights, int n,
                          int top, int width, const float* scale, cudaStream_t stream) {
  if (n <= 0 || width <= 0) return 0;
  if (width % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0)
    bw::launch_pdl(combine_kernel<true>, dim3(n, (width / 4 + 127) / 128), dim3(128), 0, stream, x, d, y, place, weights, top,
                   width, scale);
  else
    bw::launch_pdl(combine_kernel<false>, dim3(n, (width + 255) / 256), dim3(256), 0, stream, x, d, y, place, weights, top,
                   width, scale);
  return bw::launch_status();
}
