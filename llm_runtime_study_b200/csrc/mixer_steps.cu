// Small steps around attention mixers whose heads are normalised without a rotation, or that keep a
// low-rank latent per token instead of keys and values; and the norm that sits on a sublayer's output.
// Statistics, angles and gates are float32; what is stored is rounded once.
#include "common.cuh"

namespace b200 {

// ------------------------------------------------------------- per-head norm and page write
// Rows [q: nq x d | k: nkv x d | v: nkv x dv | ...].  Each q and k head is divided by its root mean
// square (eps inside the root), times q_w / k_w (d floats each) where given; q goes to q_out
// [n, nq, d], k and v into the pages [pages, nkv, page_size, d | dv] at the token's position.
// `normalise` 0 leaves q and k as they are.  The values start at column v_off of the row: (nq + nkv) * d where v has
// columns of its own; nq * d where the values are the keys as projected (before their norm; dv = d then).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_write_kernel(const T* __restrict__ rows, int ld, T* __restrict__ q_out, const float* __restrict__ q_w,
                       const float* __restrict__ k_w, float eps, int normalise, const int* __restrict__ positions,
                       const int* __restrict__ token_entry, const int* __restrict__ block_table, int table_stride,
                       int page_size, T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int d, int dv, int v_off) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* row = rows + static_cast<size_t>(token) * ld;
  const int p = positions[token];
  const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + p / page_size];
  const int in_page = p % page_size;
  for (int head = warp; head < nq + 2 * nkv; head += warps) {
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    const T* src;
    T* dst;
    int width;
    const float* w = nullptr;
    if (is_q) {
      src = row + head * d;
      dst = q_out + (static_cast<size_t>(token) * nq + head) * d;
      width = d;
      w = q_w;
    } else if (is_k) {
      const int h = head - nq;
      src = row + (nq + h) * d;
      dst = page >= 0 ? k_pool + ((static_cast<size_t>(page) * nkv + h) * page_size + in_page) * d : nullptr;
      width = d;
      w = k_w;
    } else {
      const int h = head - nq - nkv;
      src = row + v_off + h * dv;
      dst = page >= 0 ? v_pool + ((static_cast<size_t>(page) * nkv + h) * page_size + in_page) * dv : nullptr;
      width = dv;
    }
    if (dst == nullptr) continue;      // a row that pads the batch holds no page
    float f = 1.f;
    if (normalise && (is_q || is_k)) {
      float ss = 0.f;
      for (int i = lane; i < width; i += 32) {
        const float x = to_float(src[i]);
        ss = fmaf(x, x, ss);
      }
      f = rsqrtf(warp_sum(ss) / static_cast<float>(width) + eps);
    }
    for (int i = lane; i < width; i += 32) {
      float x = to_float(src[i]) * f;
      if (w != nullptr && (is_q || is_k)) x *= w[i];
      dst[i] = from_float<T>(x);
    }
  }
}

// ------------------------------------------------------------- latent attention: what is kept per token
// From one stacked projection row: the query latent cols [q_off, q_off + q_rank) RMS-normed with q_w -> cq_out
// [n, q_rank]; and, when kv_rank > 0, cols [kv_off, kv_off + kv_rank) RMS-normed with kv_w followed by `rot`
// columns of which the first rot_dims are rotated (column i pairs with i + rot_dims/2, angle p * inv_freq[i]) ->
// the page row [kv_rank + rot] of the token's position.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ rows, int ld, int q_off, int q_rank, const float* __restrict__ q_w,
                      T* __restrict__ cq_out, int kv_off, int kv_rank, const float* __restrict__ kv_w, int rot, int rot_dims,
                      const float* __restrict__ inv_freq, float eps, const int* __restrict__ positions,
                      const int* __restrict__ token_entry, const int* __restrict__ block_table, int table_stride,
                      int page_size, T* __restrict__ pool) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const T* row = rows + static_cast<size_t>(token) * ld;
  {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float x = to_float(row[q_off + i]);
      ss = fmaf(x, x, ss);
    }
    const float f = rsqrtf(block_sum(ss, scratch) / static_cast<float>(q_rank) + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      cq_out[static_cast<size_t>(token) * q_rank + i] = from_float<T>(to_float(row[q_off + i]) * f * q_w[i]);
  }
  if (kv_rank <= 0) return;
  const int p = positions[token];
  const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + p / page_size];
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float x = to_float(row[kv_off + i]);
    ss = fmaf(x, x, ss);
  }
  const float f = rsqrtf(block_sum(ss, scratch) / static_cast<float>(kv_rank) + eps);
  if (page < 0) return;
  T* dst = pool + (static_cast<size_t>(page) * page_size + p % page_size) * (kv_rank + rot);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_float<T>(to_float(row[kv_off + i]) * f * kv_w[i]);
  const int half = rot_dims / 2;
  const T* src = row + kv_off + kv_rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(static_cast<float>(p) * inv_freq[i], &sn, &cs);
    const float u = to_float(src[i]), v = to_float(src[i + half]);
    dst[kv_rank + i] = from_float<T>(u * cs - v * sn);
    dst[kv_rank + i + half] = from_float<T>(v * cs + u * sn);
  }
  for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) dst[kv_rank + i] = src[i];
}

// ------------------------------------------------------------- rotation of a slice of every head
// src rows [n, heads x src_head] : columns [src_off, src_off + rot) of every head, of which the first rot_dims are
// rotated, are written to dst rows [n, heads x dst_head] at columns [dst_off, dst_off + rot).
template <typename T>
__global__ void __launch_bounds__(128)
rope_slice_kernel(const T* __restrict__ src, int src_ld, int src_head, int src_off, T* __restrict__ dst, int dst_ld, int dst_head,
                  int dst_off, int heads, int rot, int rot_dims, const float* __restrict__ inv_freq,
                  const int* __restrict__ positions) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const float p = static_cast<float>(positions[token]);
  const int half = rot_dims / 2, per_head = half + (rot - rot_dims);
  for (int j = threadIdx.x; j < heads * per_head; j += blockDim.x) {
    const int h = j / per_head, i = j % per_head;
    const T* s = src + static_cast<size_t>(token) * src_ld + h * src_head + src_off;
    T* o = dst + static_cast<size_t>(token) * dst_ld + h * dst_head + dst_off;
    if (i < half) {
      float sn, cs;
      sincosf(p * inv_freq[i], &sn, &cs);
      const float u = to_float(s[i]), v = to_float(s[i + half]);
      o[i] = from_float<T>(u * cs - v * sn);
      o[i + half] = from_float<T>(v * cs + u * sn);
    } else {
      o[rot_dims + i - half] = s[rot_dims + i - half];
    }
  }
}

// ------------------------------------------------------------- sigmoid gate on a mixer's read-out
// out[t, c] = x[t, c] * sigmoid(gate[t, c / group]); gate rows have a stride of their own (columns of a stacked projection).
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const T* __restrict__ x, const T* __restrict__ gate, int gate_ld, int group, T* __restrict__ out, int width) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const T* g = gate + static_cast<size_t>(token) * gate_ld;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float logit = to_float(g[c / group]);
    const float s = 1.f / (1.f + expf(-logit));
    out[static_cast<size_t>(token) * width + c] = from_float<T>(to_float(x[static_cast<size_t>(token) * width + c]) * s);
  }
}

// ------------------------------------------------------------- norm on a sublayer's output
// resid[t] += x[t] * rsqrt(mean(x[t]^2) + eps) * w  (x null: nothing is added); `rounded` (optional) receives the updated
// rows in the activation type, for the sublayer that reads them next.  The sublayer's output row may be given in pieces:
// with pair_row, row t of x is sum_j pair_w[t, j] * x[pair_row[t, j]] (j ascending; what a router's experts returned for the
// token), formed here instead of by a launch of its own.  The row is kept in shared memory between the two passes.
template <typename T>
__global__ void __launch_bounds__(256)
norm_accumulate_round_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ resid,
                             T* __restrict__ rounded, int hidden, float eps, const int* __restrict__ pair_row,
                             const float* __restrict__ pair_w, int top) {
  __shared__ float scratch[32];
  extern __shared__ __align__(16) float kept[];
  pdl_trigger();
  pdl_wait();
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  float f = 0.f;
  if (x != nullptr) {
    float ss = 0.f;
    if (pair_row != nullptr) {
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
          const int p = blockIdx.x * top + j;
          acc = fmaf(pair_w[p], x[static_cast<size_t>(pair_row[p]) * hidden + i], acc);
        }
        kept[i] = acc;
        ss = fmaf(acc, acc, ss);
      }
    } else if ((hidden & 3) == 0) {
      for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(x + base)[i];
        reinterpret_cast<float4*>(kept)[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    } else {
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        kept[i] = x[base + i];
        ss = fmaf(kept[i], kept[i], ss);
      }
    }
    f = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  }
  if ((hidden & 3) == 0 && x != nullptr) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(kept)[i], g = reinterpret_cast<const float4*>(w)[i];
      float4 r = reinterpret_cast<float4*>(resid + base)[i];
      r.x += v.x * f * g.x; r.y += v.y * f * g.y; r.z += v.z * f * g.z; r.w += v.w * f * g.w;
      reinterpret_cast<float4*>(resid + base)[i] = r;
      if (rounded != nullptr) {
        rounded[base + 4 * i] = from_float<T>(r.x);
        rounded[base + 4 * i + 1] = from_float<T>(r.y);
        rounded[base + 4 * i + 2] = from_float<T>(r.z);
        rounded[base + 4 * i + 3] = from_float<T>(r.w);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float r = resid[base + i];
    if (x != nullptr) {
      r += kept[i] * f * w[i];
      resid[base + i] = r;
    }
    if (rounded != nullptr) rounded[base + i] = from_float<T>(r);
  }
}

}  // namespace b200

// v_off: the column at which the values' heads start in a row.
extern "C" int b200_head_norm_write_at(const void* rows, int ld, void* q_out, const float* q_w, const float* k_w, float eps,
                                       int normalise, const int* positions, const int* token_entry, const int* block_table,
                                       int table_stride, int page_size, void* k_pool, void* v_pool, int n, int nq, int nkv, int d,
                                       int dv, int v_off, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (nq < 0 || nkv < 0 || nq + nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || ld < (nq + nkv) * d || v_off < 0 ||
      ld < v_off + nkv * dv)
    return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(head_norm_write_kernel<T>, dim3(n), dim3(128), 0, stream, static_cast<const T*>(rows), ld,
                                       static_cast<T*>(q_out), q_w, k_w, eps, normalise, positions, token_entry, block_table,
                                       table_stride, page_size, static_cast<T*>(k_pool), static_cast<T*>(v_pool), nq, nkv, d, dv,
                                       v_off));
  return launch_status();
}

extern "C" int b200_head_norm_write(const void* rows, int ld, void* q_out, const float* q_w, const float* k_w, float eps,
                                    int normalise, const int* positions, const int* token_entry, const int* block_table,
                                    int table_stride, int page_size, void* k_pool, void* v_pool, int n, int nq, int nkv, int d,
                                    int dv, int dtype, cudaStream_t stream) {
  return b200_head_norm_write_at(rows, ld, q_out, q_w, k_w, eps, normalise, positions, token_entry, block_table, table_stride,
                                 page_size, k_pool, v_pool, n, nq, nkv, d, dv, (nq + nkv) * d, dtype, stream);
}

extern "C" int b200_latent_prepare(const void* rows, int ld, int q_off, int q_rank, const float* q_w, void* cq_out, int kv_off,
                                   int kv_rank, const float* kv_w, int rot, int rot_dims, const float* inv_freq, float eps,
                                   const int* positions, const int* token_entry, const int* block_table, int table_stride,
                                   int page_size, void* pool, int n, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (q_rank <= 0 || kv_rank < 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || q_off < 0 || q_off + q_rank > ld ||
      (kv_rank > 0 && (kv_off < 0 || kv_off + kv_rank + rot > ld || page_size <= 0)))
    return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(latent_prepare_kernel<T>, dim3(n), dim3(256), 0, stream, static_cast<const T*>(rows), ld, q_off,
                                       q_rank, q_w, static_cast<T*>(cq_out), kv_off, kv_rank, kv_w, rot, rot_dims, inv_freq, eps,
                                       positions, token_entry, block_table, table_stride, page_size, static_cast<T*>(pool)));
  return launch_status();
}

extern "C" int b200_rope_slice(const void* src, int src_ld, int src_head, int src_off, void* dst, int dst_ld, int dst_head,
                               int dst_off, int heads, int rot, int rot_dims, const float* inv_freq, const int* positions, int n,
                               int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0 || rot <= 0) return 0;
  if (heads <= 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || src_off + rot > src_head || dst_off + rot > dst_head)
    return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(rope_slice_kernel<T>, dim3(n), dim3(128), 0, stream, static_cast<const T*>(src), src_ld,
                                       src_head, src_off, static_cast<T*>(dst), dst_ld, dst_head, dst_off, heads, rot, rot_dims,
                                       inv_freq, positions));
  return launch_status();
}

extern "C" int b200_sigmoid_gate(const void* x, const void* gate, int gate_ld, int group, void* out, int n, int width, int dtype,
                                 cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || group <= 0) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(sigmoid_gate_kernel<T>, dim3(n), dim3(256), 0, stream, static_cast<const T*>(x),
                                       static_cast<const T*>(gate), gate_ld, group, static_cast<T*>(out), width));
  return launch_status();
}

extern "C" int b200_norm_accumulate_round(const float* x, const float* w, float* resid, void* rounded, int n, int hidden, float eps,
                                          const int* pair_row, const float* pair_w, int top, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (hidden <= 0 || hidden > 12288 || (pair_row != nullptr && (pair_w == nullptr || top <= 0 || x == nullptr))) return B200_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(resid)) & 15) return B200_ERR_BAD_SIZE;
  const size_t smem = x != nullptr ? sizeof(float) * hidden : 0;
  B200_DISPATCH_DTYPE(dtype, T, launch(norm_accumulate_round_kernel<T>, dim3(n), dim3(256), smem, stream, x, w, resid,
                                       static_cast<T*>(rounded), hidden, eps, pair_row, pair_w, top));
  return launch_status();
}
