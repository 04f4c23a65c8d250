// Steps of a layer whose two sublayers read one normalised copy of the stream side by side:
// layer norm (mean and variance, a weight, no bias), a short causal convolution over time added to
// what each sublayer reads (inputs before the step come from rows kept per request), the sum of the
// scaled sublayer outputs into the stream together with a weighted average over the results of all
// layers so far, a polynomial activation of normalised powers, and the gated unit of routed rows
// whose router weight multiplies the expert's input.  Statistics and sums are float32; the order of
// every sum depends on the row's width or on the token's own position only.
#include "common.cuh"

namespace b200 {

// One CTA per output row.  rows == nullptr: row r of resid (after adding delta in place when asked);
// otherwise row rows[r] is gathered and resid is left as it is.
template <typename TO>
__global__ void __launch_bounds__(256)
layer_norm_kernel(float* __restrict__ resid, const float* __restrict__ delta, const float* __restrict__ w, TO* __restrict__ out,
                  const int* __restrict__ rows, int hidden, float eps, int store_sum) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const size_t src = rows ? static_cast<size_t>(rows[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  float* x = resid + src * hidden;
  const float* dl = delta ? delta + src * hidden : nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = x[i];
    if (dl) {
      v += dl[i];
      if (store_sum) x[i] = v;
    }
    row[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float c = row[i] - mean;
    ss = fmaf(c, c, ss);
  }
  const float r = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  TO* o = out + static_cast<size_t>(blockIdx.x) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>((row[i] - mean) * r * w[i]);
}

// out_a[t, c] = h[t, c] + sum_j wa[c, j] * h[t - (K - 1) + j, c]  (and the same with wb into out_b): rows before the
// entry's first row of this step come from kept[slot] ([K - 1, C], oldest first; zeros for a new request).
template <typename TO>
__global__ void __launch_bounds__(256)
taps_pair_kernel(const float* __restrict__ h, const float* __restrict__ wa, const float* __restrict__ wb,
                 const float* __restrict__ kept, const int* __restrict__ q_start, const int* __restrict__ slots,
                 const int* __restrict__ token_entry, TO* __restrict__ out_a, TO* __restrict__ out_b, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int e = token_entry[t];
  const int first = q_start[e];
  const float* st = kept ? kept + static_cast<size_t>(slots[e]) * (K - 1) * C : nullptr;
  float a = 0.f, b = 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = t - (K - 1) + j;
    const float v = src >= first ? h[static_cast<size_t>(src) * C + c]
                                 : st[static_cast<size_t>((K - 1) - (first - src)) * C + c];
    a = fmaf(wa[static_cast<size_t>(c) * K + j], v, a);
    if (wb) b = fmaf(wb[static_cast<size_t>(c) * K + j], v, b);
  }
  const float mine = h[static_cast<size_t>(t) * C + c];
  out_a[static_cast<size_t>(t) * C + c] = from_float<TO>(mine + a);
  if (wb) out_b[static_cast<size_t>(t) * C + c] = from_float<TO>(mine + b);
}

// new = x + sa * a + sb * b is this layer's result: it is kept as results[index + 1] and the stream becomes
// sum_{j <= index + 1} mix[j] * results[j] (results: [count, n * C], results[0] the embedding's rows).
// mix == nullptr: the stream is the layer's result itself and nothing is kept.
__global__ void __launch_bounds__(256)
scale_sum_average_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ sa,
                         const float* __restrict__ b, const float* __restrict__ sb, float* __restrict__ results,
                         const float* __restrict__ mix, int index, size_t total, int C) {
  pdl_trigger();
  pdl_wait();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  float v = x[i];
  float add = (sa ? sa[c] : 1.f) * a[i];
  if (b) add += (sb ? sb[c] : 1.f) * b[i];
  v += add;
  if (mix) {
    results[static_cast<size_t>(index + 1) * total + i] = v;
    float acc = 0.f;
    for (int j = 0; j <= index; ++j) acc = fmaf(mix[j], results[static_cast<size_t>(j) * total + i], acc);
    v = fmaf(mix[index + 1], v, acc);
  }
  x[i] = v;
}

// out = c0 * z * r1 + c1 * z^2 * r2 + c2 * z^3 * r3 + c3 with r_k = rsqrt(mean over the row of z^(2k) + eps).
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const T* row = z + static_cast<size_t>(blockIdx.x) * width;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(row[i]);
    const float v2 = v * v;
    s1 += v2;
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v2 * v, v2 * v, s3);
  }
  const float n = static_cast<float>(width);
  const float r1 = rsqrtf(block_sum(s1, scratch) / n + eps);
  const float r2 = rsqrtf(block_sum(s2, scratch) / n + eps);
  const float r3 = rsqrtf(block_sum(s3, scratch) / n + eps);
  const float c0 = coef[0] * r1, c1 = coef[1] * r2, c2 = coef[2] * r3, c3 = coef[3];
  T* o = out + static_cast<size_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(row[i]);
    o[i] = from_float<T>(fmaf(c0, v, fmaf(c1, v * v, fmaf(c2, v * v * v, c3))));
  }
}

// Rows [gate | up] of width 2 F: out = silu(s * gate) * (s * up) with one factor s per row.  With pair_row the rows are
// those of (token, choice) pairs: pair p owns row pair_row[p] and its factor is scale[p]; rows no pair owns are left alone.
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_scaled_kernel(const T* __restrict__ gate_up, const int* __restrict__ pair_row, const float* __restrict__ scale,
                       T* __restrict__ out, int F) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const size_t r = pair_row ? static_cast<size_t>(pair_row[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  const float s = scale ? scale[blockIdx.x] : 1.f;
  const float g = s * to_float(gate_up[r * 2 * F + c]);
  const float u = s * to_float(gate_up[r * 2 * F + F + c]);
  out[r * F + c] = from_float<T>(g / (1.f + expf(-g)) * u);
}

}  // namespace b200

extern "C" int b200_layer_norm(float* resid, const float* delta, const float* w, void* out, const int* rows, int n, int hidden,
                               float eps, int store_sum, int out_dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (hidden <= 0) return B200_ERR_BAD_SIZE;
  const size_t smem = sizeof(float) * hidden;
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(out_dtype, TO, launch(layer_norm_kernel<TO>, dim3(n), dim3(256), smem, stream, resid, delta, w,
                                            static_cast<TO*>(out), rows, hidden, eps, store_sum));
  return launch_status();
}

extern "C" int b200_taps_pair(const float* h, const float* wa, const float* wb, const float* kept, const int* q_start,
                              const int* slots, const int* token_entry, void* out_a, void* out_b, int n, int C, int K,
                              int out_dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (C <= 0 || K <= 0 || (K > 1 && !kept)) return B200_ERR_BAD_SIZE;
  dim3 grid(n, (C + 255) / 256);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(out_dtype, TO, launch(taps_pair_kernel<TO>, grid, dim3(256), 0, stream, h, wa, wb, kept, q_start, slots,
                                            token_entry, static_cast<TO*>(out_a), static_cast<TO*>(out_b), C, K));
  return launch_status();
}

extern "C" int b200_scale_sum_average(float* x, const float* a, const float* sa, const float* b, const float* sb, float* results,
                                      const float* mix, int index, int n, int C, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (C <= 0 || index < 0) return B200_ERR_BAD_SIZE;
  const size_t total = static_cast<size_t>(n) * C;
  launch(scale_sum_average_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, x, a, sa, b, sb, results,
         mix, index, total, C);
  return launch_status();
}

extern "C" int b200_poly_norm(const void* z, const float* coef, void* out, int n, int width, float eps, int dtype,
                              cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, launch(poly_norm_kernel<T>, dim3(n), dim3(256), 0, stream, static_cast<const T*>(z), coef,
                                       static_cast<T*>(out), width, eps));
  return launch_status();
}

extern "C" int b200_silu_mul_scaled(const void* gate_up, const int* pair_row, const float* scale, void* out, int rows, int F,
                                    int dtype, cudaStream_t stream) {
  using namespace b200;
  if (rows <= 0) return 0;
  if (F <= 0) return B200_ERR_BAD_SIZE;
  dim3 grid(rows, (F + 255) / 256);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, launch(silu_mul_scaled_kernel<T>, grid, dim3(256), 0, stream, static_cast<const T*>(gate_up),
                                       pair_row, scale, static_cast<T*>(out), F));
  return launch_status();
}
