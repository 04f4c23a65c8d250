// Causal attention over the paged cache on CUDA cores, 32-bit arithmetic throughout.
// It serves prompt portions and single decoded tokens alike: every query token is
// handled by itself (one warp per token and query head), reading keys 0..p of its
// request through the block table, in tiles of 32 keys that start at key 0.  The
// order of every sum is therefore a function of the token's own position only, so a
// token's output is bit-identical however the batch was cut.
//
// Formula (mini_llm/nn/attention.py:95-99, 231-248): S = q.k^T * scale, key t visible
// iff t <= p (and t > p - window when a window is set), P = softmax(S), o = P.v;
// query head j reads KV head j / (nq / nkv)  (mini_llm/nn/attention.py:18-33).
//
// Optional rules on the scores, each a parameter: a soft cap (S <- cap * tanh(S / cap)), a
// bias by distance (S <- S - slope_j * (p - t) with one slope per query head), and a sink
// (a virtual key of score 0 that carries no value: the weights become exp(S) / (1 + sum exp(S))).
// Values may have a head size `dv` of their own.  Two further rules: a bias by the logarithm of the distance
// (S <- S - r1_j * ln(1 + r2_j * (p - t)) with two numbers per query head) and a mask in blocks (`chunk` > 0: position p
// sees t only if floor(p / chunk) = floor(t / chunk), blocks counted from position 0 of the sequence).
#include "common.cuh"

namespace b200 {

// kMaxChunks x 32 columns of values at most; the key size is bounded by shared memory only
template <typename T, int kMaxChunks>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                            const T* __restrict__ v_pool, T* __restrict__ out,
                            const int* __restrict__ positions, const int* __restrict__ token_entry,
                            const int* __restrict__ block_table, int table_stride, int page_size,
                            int nq, int nkv, int d, float scale, int window, int dv, float softcap,
                            const float* __restrict__ slopes, int sink, int v_row, int chunk,
                            const float* __restrict__ log_r1, const float* __restrict__ log_r2) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int head = blockIdx.y * 4 + warp;
  if (head >= nq) return;
  const int kvh = head / (nq / nkv);
  const int p = positions[token];
  const int* table = block_table + static_cast<size_t>(token_entry[token]) * table_stride;
  float* qs = smem + warp * d;
  const T* qrow = q + (static_cast<size_t>(token) * nq + head) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qrow[i]);
  __syncwarp();

  int w0 = window > 0 ? max(0, p - window + 1) : 0;
  if (chunk > 0) w0 = max(w0, p / chunk * chunk);
  // the sink is a key of score 0 and value 0 that every row sees: it starts the running maximum and sum
  float m = sink ? 0.f : -INFINITY, l = sink ? 1.f : 0.f;
  const float slope = slopes ? slopes[head] : 0.f;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const float r1 = log_r1 ? log_r1[head] : 0.f, r2 = log_r2 ? log_r2[head] : 0.f;
  float acc[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) acc[c] = 0.f;

  constexpr int VN = Vec<T>::n;
  for (int t0 = (w0 / 32) * 32; t0 <= p; t0 += 32) {
    const int t = t0 + lane;
    bool valid = t <= p && t >= w0;
    float s = -INFINITY;
    const int page = valid ? table[t / page_size] : -1;
    valid = valid && page >= 0;      // a page given back (window) or a padding row without pages
    if (valid) {
      const T* krow = k_pool + ((static_cast<size_t>(page) * nkv + kvh) * page_size + t % page_size) * d;
      float dot = 0.f;
      if (d % VN == 0) {         // rows of keys then start on 16-byte boundaries
        for (int i = 0; i < d; i += VN) {
          float f[VN];
          Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::type*>(krow + i), f);
#pragma unroll
          for (int e = 0; e < VN; ++e) dot = fmaf(qs[i + e], f[e], dot);
        }
      } else {
        for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_float(krow[i]), dot);
      }
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
      s -= slope * static_cast<float>(p - t);
      if (log_r1 != nullptr) s -= r1 * log1pf(r2 * static_cast<float>(p - t));
    }
    const float m_tile = warp_max(s);
    if (m_tile == -INFINITY) continue;
    const float m_new = fmaxf(m, m_tile);
    const float corr = expf(m - m_new);  // m = -inf -> 0
    const float pl = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) acc[c] *= corr;
    const int count = min(32, p - t0 + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pl, j);
      if (pj == 0.f) continue;
      const int tj = t0 + j;
      const int page = table[tj / page_size];
      const T* vrow = v_pool + ((static_cast<size_t>(page) * nkv + kvh) * page_size + tj % page_size) * v_row;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
      }
    }
    m = m_new;
  }
  T* orow = out + (static_cast<size_t>(token) * nq + head) * dv;
  const float inv = l > 0.f ? 1.f / l : 0.f;   // a row without any visible key (padding) gives zeros
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) orow[i] = from_float<T>(acc[c] * inv);
  }
}

}  // namespace b200

// q [n, nq, d], keys [pages, nkv, page_size, d], values [pages, nkv, page_size, v_row] of which the first dv columns are read
// (v_row = dv: a pool of its own; v_row = d with v_pool = k_pool: the values are the leading columns of the keys),
// out [n, nq, dv].  softcap <= 0: no cap; slopes (nq floats) may be null; sink 0 or 1.
extern "C" int b200_paged_attention_simt_strided(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, int dv, int v_row, float scale, int window, float softcap, const float* slopes, int sink,
    int dtype, cudaStream_t stream);

// The same with the mask in blocks (chunk <= 0: none) and the bias by the logarithm of the distance (log_r1, log_r2:
// [nq] floats each, or both null).
extern "C" int b200_paged_attention_simt_masked(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, int dv, int v_row, float scale, int window, float softcap, const float* slopes, int sink,
    int chunk, const float* log_r1, const float* log_r2, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (d <= 0 || dv <= 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || v_row < dv ||
      (log_r1 == nullptr) != (log_r2 == nullptr))
    return B200_ERR_BAD_SIZE;
  if (dv > 32 * 20 || d > 2048) return B200_ERR_TOO_LARGE;
  dim3 grid(n, (nq + 3) / 4);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  const size_t smem = static_cast<size_t>(4) * d * sizeof(float);
#define B200_SIMT_ATTENTION(CH)                                                                             \
  B200_DISPATCH_DTYPE(dtype, T,                                                                             \
      launch(paged_attention_simt_kernel<T, CH>, dim3(grid), dim3(128), smem, stream,                       \
          static_cast<const T*>(q), static_cast<const T*>(k_pool), static_cast<const T*>(v_pool),          \
          static_cast<T*>(out), positions, token_entry, block_table, table_stride, page_size, nq,           \
          nkv, d, scale, window, dv, softcap, slopes, sink, v_row, chunk, log_r1, log_r2))
  if (dv <= 64) { B200_SIMT_ATTENTION(2); }
  else if (dv <= 128) { B200_SIMT_ATTENTION(4); }
  else if (dv <= 256) { B200_SIMT_ATTENTION(8); }
  else { B200_SIMT_ATTENTION(20); }
#undef B200_SIMT_ATTENTION
  return launch_status();
}

extern "C" int b200_paged_attention_simt_strided(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, int dv, int v_row, float scale, int window, float softcap, const float* slopes, int sink,
    int dtype, cudaStream_t stream) {
  return b200_paged_attention_simt_masked(q, k_pool, v_pool, out, positions, token_entry, block_table, table_stride, page_size,
                                          n, nq, nkv, d, dv, v_row, scale, window, softcap, slopes, sink, 0, nullptr, nullptr,
                                          dtype, stream);
}

extern "C" int b200_paged_attention_simt_rules(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, int dv, float scale, int window, float softcap, const float* slopes, int sink,
    int dtype, cudaStream_t stream) {
  if (d > 256 || dv > 256) return B200_ERR_TOO_LARGE;
  return b200_paged_attention_simt_strided(q, k_pool, v_pool, out, positions, token_entry, block_table, table_stride, page_size,
                                           n, nq, nkv, d, dv, dv, scale, window, softcap, slopes, sink, dtype, stream);
}

extern "C" int b200_paged_attention_simt(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, float scale, int window, int dtype, cudaStream_t stream) {
  return b200_paged_attention_simt_rules(q, k_pool, v_pool, out, positions, token_entry, block_table, table_stride,
                                         page_size, n, nq, nkv, d, d, scale, window, 0.f, nullptr, 0, dtype, stream);
}
