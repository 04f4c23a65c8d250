// Matrix products in groups: one weight per batch index (heads, diagonal blocks), or one weight per group of rows
// that a router has sent to the same expert.  C = A * W^T (+ bias), float accumulation in ascending k inside one
// thread, so a row's result depends neither on the other rows of the batch nor on where the row sits in its tile.
// Storage types float32 (FFMA only: the verification path) and bfloat16: on the tensor cores (mma.sync m16n8k16, tiles
// staged by cp.async in three stages) where rows and strides are multiples of 16 bytes, on CUDA cores otherwise.
// Also the router of a mixture of experts and the bookkeeping that sorts
// (token, choice) pairs by expert without the host knowing the counts.
#include "common.cuh"
#include "mma.cuh"

namespace b200 {

constexpr int BM = 64, BN = 64, BK = 16;

struct GroupedArgs {
  const void* A; long long lda, a_z;        // rows of A; a_z: elements between batch entries
  const int* row_index;                     // per row of the tile space: source row or validity (< 0: the row is padding)
  int gather;                               // 1: row_index names the row of A; 0: row m of A is used, row_index only says valid
  const void* W; long long ldw, w_z;        // W[z]: [N, K] with row stride ldw, or (k_major) [K, N]
  int k_major;
  const float* bias; long long bias_z;
  void* C; long long ldc, c_z;
  const int* tile_group;                    // per row tile: the group (expert) whose weight it uses, < 0: nothing to do
  int group_tile_rows;                      // rows of the tiles tile_group speaks of (a multiple of BM)
  int M, N, K;
};

template <typename TIn, typename TOut, int ACT>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const GroupedArgs g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int src_row[BM];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int z = blockIdx.z;
  long long a_off = z * g.a_z, c_off = z * g.c_z;
  if (g.tile_group != nullptr) {
    z = g.tile_group[blockIdx.y * BM / g.group_tile_rows];
    if (z < 0) return;
    a_off = c_off = 0;
  }
  const TIn* A = static_cast<const TIn*>(g.A) + a_off;
  const TIn* W = static_cast<const TIn*>(g.W) + z * g.w_z;
  const float* bias = g.bias ? g.bias + z * g.bias_z : nullptr;
  TOut* C = static_cast<TOut*>(g.C) + c_off;
  if (tid < BM) {
    const int m = m0 + tid;
    int r = m < g.M ? m : -1;
    if (r >= 0 && g.row_index != nullptr) {
      const int v = g.row_index[m];
      r = v < 0 ? -1 : (g.gather ? v : m);
    }
    src_row[tid] = r;
  }
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4] = {};
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int arow = src_row[lrow];
  const int wn = n0 + lrow;
  for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lrow] = (arow >= 0 && k < g.K) ? to_float(A[arow * g.lda + k]) : 0.f;
      float w = 0.f;
      if (wn < g.N && k < g.K) w = to_float(g.k_major ? W[k * g.ldw + wn] : W[wn * g.ldw + k]);
      Ws[lk + i][lrow] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (src_row[ty * 4 + i] < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j] + (bias ? bias[n] : 0.f);
      if (ACT == 1) {          // the square of relu
        v = fmaxf(v, 0.f);
        v *= v;
      }
      C[m * g.ldc + n] = from_float<TOut>(v);
    }
  }
}

// ----------------------------------------------------------------------------- bfloat16 on the tensor cores
// The same tile space (BM rows of one group or batch entry) with BN = 128 columns and BK = 64 per stage, four stages
// (110 KB in flight per CTA: what a few rows against a large weight need to stream it).  Eight warps,
// two along the rows and four along the columns, each 32 x 32 outputs.  Every 16-byte chunk of A and W must start on a
// 16-byte boundary: base pointers, row strides and batch strides are multiples of 8 elements (the launcher checks).
constexpr int TBK = 64, TPAD = 8, TSTAGES = 4;
constexpr int TLD = TBK + TPAD;                         // 72 halves = 144 bytes a row: ldmatrix reads hit every bank once

// TBN columns a tile: 128, or 64 for launches of few tiles (single tokens against large weights), which then have twice the
// CTAs and two of them on a multiprocessor.
template <typename TOut, int ACT, int TBN>
__global__ void __launch_bounds__(256)
grouped_gemm_mma_kernel(const GroupedArgs g) {
  constexpr int TSTAGE_HALVES = (BM + TBN) * TLD;
  constexpr int WN = TBN / 4;             // columns of a warp
  constexpr int NB = WN / 16;             // B fragments (16 columns each) a k step
  constexpr int NJ = WN / 8;              // 8-column accumulator tiles
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ int src_row[BM];
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * TBN;
  pdl_wait();
  int z = blockIdx.z;
  long long a_off = z * g.a_z, c_off = z * g.c_z;
  if (g.tile_group != nullptr) {
    z = g.tile_group[blockIdx.y * BM / g.group_tile_rows];
    if (z < 0) return;
    a_off = c_off = 0;
  }
  const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(g.A) + a_off;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(g.W) + z * g.w_z;
  const float* bias = g.bias ? g.bias + z * g.bias_z : nullptr;
  TOut* C = static_cast<TOut*>(g.C) + c_off;
  if (tid < BM) {
    const int m = m0 + tid;
    int r = m < g.M ? m : -1;
    if (r >= 0 && g.row_index != nullptr) {
      const int v = g.row_index[m];
      r = v < 0 ? -1 : (g.gather ? v : m);
    }
    src_row[tid] = r;
  }
  __syncthreads();
  // chunks of 8 halves: A has BM x 8 of them (two a thread), W has TBN x 8 (four a thread)
  auto stage_load = [&](int stage, int k0) {
    __nv_bfloat16* As = tiles + stage * TSTAGE_HALVES;
    __nv_bfloat16* Ws = As + BM * TLD;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * 256;
      const int a_row = c >> 3, a_chunk = (c & 7) * 8;
      const int a_src = src_row[a_row];
      const int k = k0 + a_chunk;
      const int bytes = a_src >= 0 ? max(0, min(16, (g.K - k) * 2)) : 0;
      const __nv_bfloat16* src = bytes > 0 ? A + a_src * g.lda + k : A;
      cp_async_16(As + a_row * TLD + a_chunk, src, bytes);
    }
#pragma unroll
    for (int i = 0; i < TBN / 32; ++i) {
      const int c = tid + i * 256;
      const int row = c >> 3, chunk = (c & 7) * 8;
      const int n = n0 + row, k = k0 + chunk;
      const int bytes = n < g.N ? max(0, min(16, (g.K - k) * 2)) : 0;
      const __nv_bfloat16* src = bytes > 0 ? W + n * g.ldw + k : W;
      cp_async_16(Ws + row * TLD + chunk, src, bytes);
    }
  };
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * WN;
  float acc[2][NJ][4] = {};
  const int k_tiles = (g.K + TBK - 1) / TBK;
#pragma unroll
  for (int s = 0; s < TSTAGES - 1; ++s) {
    if (s < k_tiles) stage_load(s, s * TBK);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<TSTAGES - 2>();
    __syncthreads();
    if (kt + TSTAGES - 1 < k_tiles) stage_load((kt + TSTAGES - 1) % TSTAGES, (kt + TSTAGES - 1) * TBK);
    cp_async_commit();
    const __nv_bfloat16* As = tiles + (kt % TSTAGES) * TSTAGE_HALVES;
    const __nv_bfloat16* Ws = As + BM * TLD;
#pragma unroll
    for (int kk = 0; kk < TBK; kk += 16) {
      uint32_t a[2][4], b[NB][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(a[i], As + (wm + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * TLD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < NB; ++j)
        ldmatrix_x4(b[j], Ws + (wn + j * 16 + (lane & 7) + (lane >> 4) * 8) * TLD + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j) mma_bf16(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int local = wm + i * 16 + (lane >> 2) + half * 8;
      if (src_row[local] < 0) continue;
      const long long m = m0 + local;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int n = n0 + wn + j * 8 + (lane & 3) * 2 + e;
          if (n >= g.N) continue;
          float v = acc[i][j][half * 2 + e] + (bias ? bias[n] : 0.f);
          if (ACT == 1) {
            v = fmaxf(v, 0.f);
            v *= v;
          }
          C[m * g.ldc + n] = from_float<TOut>(v);
        }
    }
}

template <typename TOut, int ACT, int TBN>
int launch_grouped_mma_tile(const GroupedArgs& g, int batch, cudaStream_t stream) {
  dim3 grid((g.N + TBN - 1) / TBN, (g.M + BM - 1) / BM, batch);
  if (grid.y > 65535 || grid.z > 65535) return B200_ERR_TOO_LARGE;
  constexpr size_t smem = sizeof(__nv_bfloat16) * TSTAGES * (BM + TBN) * TLD;
  static DeviceOnce once;
  if (int e = configure_once(once, grouped_gemm_mma_kernel<TOut, ACT, TBN>, smem)) return e;
  launch(grouped_gemm_mma_kernel<TOut, ACT, TBN>, grid, dim3(256), smem, stream, g);
  return launch_status();
}

template <typename TOut>
int launch_grouped_mma(const GroupedArgs& g, int batch, int act, cudaStream_t stream) {
  // fewer tiles of 128 columns than multiprocessors (a B200 has 148): tiles of 64 columns
  const long tiles = static_cast<long>((g.N + 127) / 128) * ((g.M + BM - 1) / BM) * batch;
  const bool narrow = tiles < 148 && g.N > 64;
  if (act == 1) return narrow ? launch_grouped_mma_tile<TOut, 1, 64>(g, batch, stream) : launch_grouped_mma_tile<TOut, 1, 128>(g, batch, stream);
  return narrow ? launch_grouped_mma_tile<TOut, 0, 64>(g, batch, stream) : launch_grouped_mma_tile<TOut, 0, 128>(g, batch, stream);
}

// ----------------------------------------------------------------------------- router
// One CTA of 128 threads per token: logits z = W_r h + b in float32 (W_r float32 [experts, width], h in the activation type),
// the `top` largest (the lower index wins a tie), weights = softmax over the chosen logits only.  Every thread sums its
// share of the row for eight experts at a time; the shares meet in a warp's shuffle tree and then warp by warp in order, so
// a token's logits do not depend on the batch around it.
//
// score 2: s = softmax(z) over all outputs; the choice goes by s + correction (a float per output, may be null); the outputs
// form `groups` equal groups of neighbours, a group scores the largest choice score in it, and only outputs of the `keep`
// best groups can be chosen (the lower index wins a tie, as everywhere); weights = s (without the correction) * scale.
// The router's matrix may hold `extra` further rows behind those of the outputs (one number per token each: a gate on
// something that runs for every token); their logits' sigmoids go to extra_out [n, extra] and take no part in the choice.
// A CTA takes TOK tokens (batches of many tokens: the router's rows are fetched once for all of them); a token's sums are
// formed in the same order whatever TOK is, so its logits carry the same bits in every batch.  Warp w then chooses for the
// CTA's token w.
template <typename T, int TOK>
__global__ void __launch_bounds__(128)
route_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ br, int* __restrict__ ids,
             float* __restrict__ wts, int n, int width, int outputs, int top, int score, const float* __restrict__ correction, int groups,
             int keep, float scale, int extra, float* __restrict__ extra_out) {
  // per token: [experts] logits, [outputs] probabilities, [groups] scores; then [TOK][4][8] partial sums
  extern __shared__ float route_smem[];
  const int experts = outputs + extra;       // rows of the router's matrix
  const int per_token = experts + outputs + groups;
  float* part = route_smem + TOK * per_token;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token0 = blockIdx.x * TOK;
  const T* rows[TOK];
#pragma unroll
  for (int k = 0; k < TOK; ++k) rows[k] = h + static_cast<size_t>(min(token0 + k, n - 1)) * width;
  for (int e0 = 0; e0 < experts; e0 += 8) {
    float dot[TOK][8];
#pragma unroll
    for (int k = 0; k < TOK; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) dot[k][j] = 0.f;
    if ((width & 3) == 0) {          // four columns a thread and pass: 16-byte loads of the router's rows
      for (int i = threadIdx.x * 4; i < width; i += 512) {
        float x[TOK][4];
#pragma unroll
        for (int k = 0; k < TOK; ++k)
#pragma unroll
          for (int c = 0; c < 4; ++c) x[k][c] = to_float(rows[k][i + c]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < experts) {
            const float4 w4 = *reinterpret_cast<const float4*>(wr + static_cast<size_t>(e0 + j) * width + i);
#pragma unroll
            for (int k = 0; k < TOK; ++k)
              dot[k][j] = fmaf(x[k][3], w4.w, fmaf(x[k][2], w4.z, fmaf(x[k][1], w4.y, fmaf(x[k][0], w4.x, dot[k][j]))));
          }
      }
    } else {
      for (int i = threadIdx.x; i < width; i += 128) {
        float x[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) x[k] = to_float(rows[k][i]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < experts) {
            const float w = wr[static_cast<size_t>(e0 + j) * width + i];
#pragma unroll
            for (int k = 0; k < TOK; ++k) dot[k][j] = fmaf(x[k], w, dot[k][j]);
          }
      }
    }
#pragma unroll
    for (int k = 0; k < TOK; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sum = warp_sum(dot[k][j]);
        if (lane == 0) part[(k * 4 + warp) * 8 + j] = sum;
      }
    __syncthreads();
    if (threadIdx.x < TOK * 8 && e0 + (threadIdx.x & 7) < experts) {
      const int k = threadIdx.x >> 3, j = threadIdx.x & 7;
      const float* p = part + k * 32;
      route_smem[k * per_token + e0 + j] = ((p[j] + p[8 + j]) + p[16 + j]) + p[24 + j] + (br ? br[e0 + j] : 0.f);
    }
    __syncthreads();
  }
  if (warp >= TOK || token0 + warp >= n) return;
  const int token = token0 + warp;
  float* logits = route_smem + warp * per_token;
  float* probs = logits + experts;
  float* group_score = probs + outputs;
  if (lane < extra) extra_out[static_cast<size_t>(token) * extra + lane] = 1.f / (1.f + expf(-logits[outputs + lane]));
  if (score == 2) {
    float mx = -INFINITY;
    for (int e = lane; e < outputs; e += 32) mx = fmaxf(mx, logits[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) {
      const float p = expf(logits[e] - mx);
      probs[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < outputs; e += 32) {
      const float p = probs[e] / sum;
      probs[e] = p;
      logits[e] = p + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (groups > 1) {
      const int per = outputs / groups;
      for (int g = lane; g < groups; g += 32) {
        float best = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, logits[e]);
        group_score[g] = best;
      }
      __syncwarp();
      for (int j = 0; j < keep; ++j) {          // the kept groups are marked by +infinity
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int g = lane; g < groups; g += 32) {
          const float v = group_score[g];
          if (v != INFINITY && v > best) { best = v; at = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, at, o);
          if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        __syncwarp();
        if (lane == 0 && at < groups) group_score[at] = INFINITY;
        __syncwarp();
      }
      for (int e = lane; e < outputs; e += 32)
        if (group_score[e / per] != INFINITY) logits[e] = -INFINITY;
      __syncwarp();
    }
  }
  float first = 0.f, total = 0.f, mine = 0.f, mine_logit = 0.f;
  int my_id = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32) {
      const float v = logits[e];
      if (v > best) { best = v; at = e; }       // ascending e: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (j == 0) first = best;
    const float p = expf(best - first);
    total += p;
    if (lane == j) { mine = p; mine_logit = best; my_id = at; }
    __syncwarp();
    if (lane == 0 && at < outputs) logits[at] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    my_id = min(my_id, outputs - 1);          // nothing left to choose from (every score NaN): still a valid output
    ids[static_cast<size_t>(token) * top + lane] = my_id;
    // score 0: the softmax over the chosen logits; 1: each chosen logit's own sigmoid (the order of sigmoids is the logits');
    // 2: the chosen output's share of the softmax over all outputs, times scale
    float w = mine / total;
    if (score == 1) w = 1.f / (1.f + expf(-mine_logit));
    if (score == 2) w = probs[my_id] * scale;
    wts[static_cast<size_t>(token) * top + lane] = w;
  }
}

// One CTA.  Counts the pairs of every expert, lays the experts' rows out one behind the other, each padded to whole
// tiles of BM rows, and gives every pair its row: sorted_token[row] = token (-1 in the padding), pair_row[pair] = row,
// tile_group[tile] = expert (-1 behind the last used tile).  A tile has tile_rows rows (what the product kernel takes).
// A pair whose id is `experts` or more (a router output without an expert behind it) gets no row: pair_row = -1.
__global__ void __launch_bounds__(1024)
plan_kernel(const int* __restrict__ ids, int pairs, int top, int experts, int* __restrict__ sorted_token, int* __restrict__ pair_row,
            int* __restrict__ tile_group, int max_tiles, int tile_rows) {
  extern __shared__ int sh[];
  int* count = sh;                 // [experts]
  int* start = sh + experts;       // [experts + 1], in rows
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  for (int r = threadIdx.x; r < max_tiles * tile_rows; r += blockDim.x) sorted_token[r] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x)
    if (ids[p] < experts) atomicAdd(&count[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
      count[e] = 0;
    }
    start[experts] = at;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * tile_rows;
    int group = -1;
    if (row < start[experts]) {
      int lo = 0, hi = experts - 1;          // the last expert whose start is <= row and that has rows
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (start[mid] <= row) lo = mid; else hi = mid - 1;
      }
      group = lo;
    }
    tile_group[t] = group;
  }
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= experts) { pair_row[p] = -1; continue; }
    const int row = start[e] + atomicAdd(&count[e], 1);
    sorted_token[row] = p / top;
    pair_row[p] = row;
  }
}

// out[t] = sum_j wts[t, j] * rows[pair_row[t, j]], j ascending.
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ rows, const int* __restrict__ pair_row, const float* __restrict__ wts, float* __restrict__ out,
               int width, int top) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int p = token * top + j;
      acc = fmaf(wts ? wts[p] : 1.f, rows[static_cast<size_t>(pair_row[p]) * width + c], acc);
    }
    out[static_cast<size_t>(token) * width + c] = acc;
  }
}

// The same where a pair may have no row (pair_row < 0: the router output returns the token's own input row x[t]) and a
// further row per token is added with a factor of its own: out[t] = sum_j wts[t, j] * (rows[pair_row[t, j]] or x[t]) +
// extra_scale[t] * extra[t].  x in the activation type; extra float32 or null.
template <typename T>
__global__ void __launch_bounds__(256)
combine_mixed_kernel(const float* __restrict__ rows, const int* __restrict__ pair_row, const float* __restrict__ wts,
                     const T* __restrict__ x, const float* __restrict__ extra, const float* __restrict__ extra_scale,
                     float* __restrict__ out, int width, int top) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const float es = extra != nullptr ? extra_scale[token] : 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int p = token * top + j;
      const int r = pair_row[p];
      const float v = r >= 0 ? rows[static_cast<size_t>(r) * width + c] : to_float(x[static_cast<size_t>(token) * width + c]);
      acc = fmaf(wts[p], v, acc);
    }
    if (extra != nullptr) acc = fmaf(es, extra[static_cast<size_t>(token) * width + c], acc);
    out[static_cast<size_t>(token) * width + c] = acc;
  }
}

__global__ void __launch_bounds__(128)
gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ sorted_token, uint4* __restrict__ out, int chunks) {
  pdl_trigger();
  pdl_wait();
  const int src = sorted_token[blockIdx.x];
  for (int i = threadIdx.x; i < chunks; i += blockDim.x)
    out[static_cast<size_t>(blockIdx.x) * chunks + i] = src >= 0 ? x[static_cast<size_t>(src) * chunks + i] : make_uint4(0, 0, 0, 0);
}

template <typename TIn, typename TOut>
int launch_grouped(const GroupedArgs& g, int batch, int act, cudaStream_t stream) {
  dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, batch);
  if (grid.y > 65535 || grid.z > 65535) return B200_ERR_TOO_LARGE;
  if (act == 1) launch(grouped_gemm_kernel<TIn, TOut, 1>, grid, dim3(256), 0, stream, g);
  else launch(grouped_gemm_kernel<TIn, TOut, 0>, grid, dim3(256), 0, stream, g);
  return launch_status();
}

// LLM_RUNTIME_STUDY_B200_GROUPED=simt keeps bfloat16 products on the CUDA cores (for comparisons)
inline bool use_tensor_cores() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("LLM_RUNTIME_STUDY_B200_GROUPED");
    on = (e != nullptr && e[0] == 's') ? 0 : 1;
  }
  return on == 1;
}

}  // namespace b200

// in_dtype: storage type of A and W; out_dtype: of C.  batch > 1 walks a_z / w_z / bias_z / c_z; with tile_group the
// weight of a row tile is W + tile_group[tile] * w_z instead (batch must be 1; tile_group speaks of tiles of group_tile_rows rows).  act: 0 none, 1 relu squared.
extern "C" int b200_gemm_grouped(const void* A, long long lda, long long a_z, const int* row_index, int gather, const void* W,
                                 long long ldw, long long w_z, int k_major, const float* bias, long long bias_z, void* C,
                                 long long ldc, long long c_z, const int* tile_group, int group_tile_rows, int M, int N, int K, int batch,
                                 int act, int in_dtype, int out_dtype, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (K <= 0 || (tile_group != nullptr && (batch != 1 || group_tile_rows <= 0 || group_tile_rows % BM != 0))) return B200_ERR_BAD_SIZE;
  GroupedArgs g{A, lda, a_z, row_index, gather, W, ldw, w_z, k_major, bias, bias_z, C, ldc, c_z, tile_group, group_tile_rows, M, N, K};
  const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) == 0 && lda % 8 == 0 && a_z % 8 == 0 &&
                       ldw % 8 == 0 && w_z % 8 == 0;
  if (in_dtype == kBF16 && aligned && !k_major && use_tensor_cores()) {
    if (out_dtype == kBF16) return launch_grouped_mma<__nv_bfloat16>(g, batch, act, stream);
    if (out_dtype == kF32) return launch_grouped_mma<float>(g, batch, act, stream);
  }
  if (in_dtype == kF32 && out_dtype == kF32) return launch_grouped<float, float>(g, batch, act, stream);
  if (in_dtype == kBF16 && out_dtype == kBF16) return launch_grouped<__nv_bfloat16, __nv_bfloat16>(g, batch, act, stream);
  if (in_dtype == kBF16 && out_dtype == kF32) return launch_grouped<__nv_bfloat16, float>(g, batch, act, stream);
  return B200_ERR_BAD_DTYPE;
}

// wr float32 [outputs + extra, width]; score 0, 1 or 2 (see route_kernel); correction [outputs] or null; extra_out [n, extra].
extern "C" int b200_moe_route_grouped(const void* h, const float* wr, const float* br, const float* correction, int* ids, float* wts,
                                      float* extra_out, int n, int width, int outputs, int top, int score, int groups, int keep,
                                      float scale, int extra, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || outputs <= 0 || top <= 0 || top > outputs || top > 32 || outputs > 2048 || extra < 0 || extra > 32 ||
      (extra > 0 && extra_out == nullptr) || groups <= 0 || outputs % groups != 0 || keep <= 0 || keep > groups ||
      top > keep * (outputs / groups) || score < 0 || score > 2 || (groups > 1 && score != 2))
    return B200_ERR_BAD_SIZE;
  // many tokens: four a CTA, one choosing warp each (the router's rows cross the L2 a quarter as often)
  const bool four = n >= 512;
  const int tok = four ? 4 : 1;
  const size_t smem = sizeof(float) * tok * (outputs + extra + outputs + groups + 32);
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, {
    if (four) launch(route_kernel<T, 4>, dim3((n + 3) / 4), dim3(128), smem, stream, static_cast<const T*>(h), wr, br, ids, wts, n, width,
                     outputs, top, score, correction, groups, keep, scale, extra, extra_out);
    else launch(route_kernel<T, 1>, dim3(n), dim3(128), smem, stream, static_cast<const T*>(h), wr, br, ids, wts, n, width, outputs, top,
                score, correction, groups, keep, scale, extra, extra_out);
  });
  return launch_status();
}

extern "C" int b200_moe_route(const void* h, const float* wr, const float* br, int* ids, float* wts, int n, int width, int experts,
                              int top, int score, int dtype, cudaStream_t stream) {
  if (score < 0 || score > 1) return B200_ERR_BAD_SIZE;
  return b200_moe_route_grouped(h, wr, br, nullptr, ids, wts, nullptr, n, width, experts, top, score, 1, 1, 1.f, 0, dtype, stream);
}

extern "C" int b200_moe_tile_rows() { return b200::BM; }

extern "C" int b200_moe_plan(const int* ids, int pairs, int top, int experts, int* sorted_token, int* pair_row, int* tile_group,
                             int max_tiles, int tile_rows, cudaStream_t stream) {
  using namespace b200;
  if (pairs <= 0) return 0;
  if (experts <= 0 || experts > 2048 || top <= 0 || tile_rows <= 0 || tile_rows % BM != 0 || max_tiles * tile_rows < pairs) return B200_ERR_BAD_SIZE;
  launch(plan_kernel, dim3(1), dim3(1024), sizeof(int) * (2 * experts + 1), stream, ids, pairs, top, experts, sorted_token, pair_row,
         tile_group, max_tiles, tile_rows);
  return launch_status();
}

// out[row] = x[sorted_token[row]] (zeros where the row is padding): the rows of every expert one behind the other, for a
// product kernel that fetches its row operand by TMA.  width is a multiple of 8.
extern "C" int b200_gather_rows_bf16(const void* x, const int* sorted_token, void* out, int rows, int width, cudaStream_t stream) {
  using namespace b200;
  if (rows <= 0) return 0;
  if (width <= 0 || width % 8 != 0) return B200_ERR_BAD_SIZE;
  launch(gather_rows_kernel, dim3(rows), dim3(128), 0, stream, static_cast<const uint4*>(x), sorted_token, static_cast<uint4*>(out), width / 8);
  return launch_status();
}

extern "C" int b200_moe_combine_mixed(const float* rows, const int* pair_row, const float* wts, const void* x, const float* extra,
                                      const float* extra_scale, float* out, int n, int width, int top, int dtype,
                                      cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || top <= 0 || x == nullptr || wts == nullptr || (extra != nullptr && extra_scale == nullptr)) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(combine_mixed_kernel<T>, dim3(n), dim3(256), 0, stream, rows, pair_row, wts,
                                       static_cast<const T*>(x), extra, extra_scale, out, width, top));
  return launch_status();
}

extern "C" int b200_moe_combine(const float* rows, const int* pair_row, const float* wts, float* out, int n, int width, int top,
                                cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || top <= 0) return B200_ERR_BAD_SIZE;
  launch(combine_kernel, dim3(n), dim3(256), 0, stream, rows, pair_row, wts, out, width, top);
  return launch_status();
}
