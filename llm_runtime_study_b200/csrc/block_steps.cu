// Steps of a layer whose two sublayers read one normalised copy of the stream side by side:
// layer norm (mean and variance, a weight, no bias), a short causal convolution over time added to
// what each sublayer reads (inputs before the step come from rows kept per request), the sum of the
// scaled sublayer outputs into the stream together with a weighted average over the results of all
// layers so far, a polynomial activation of normalised powers, and the gated unit of routed rows
// whose router weight multiplies the expert's input.  Statistics and sums are float32; the order of
// every sum depends on the row's width or on the token's own position only.
#include "common.cuh"

namespace b200 {

// Four neighbouring values in one store (16 bytes of float, 8 of bfloat16); the address is a multiple of that.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  uint2 v;
  *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = v;
}

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

// The same with 16-byte accesses: hidden is a multiple of 4 and every row starts on a 16-byte boundary.
template <typename TO>
__global__ void __launch_bounds__(256)
layer_norm_vec_kernel(float* __restrict__ resid, const float* __restrict__ delta, const float* __restrict__ w, TO* __restrict__ out,
                      const int* __restrict__ rows, int hidden, float eps, int store_sum) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const size_t src = rows ? static_cast<size_t>(rows[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  float4* x = reinterpret_cast<float4*>(resid + src * hidden);
  const float4* dl = delta ? reinterpret_cast<const float4*>(delta + src * hidden) : nullptr;
  float4* row4 = reinterpret_cast<float4*>(row);
  const int quads = hidden >> 2;
  float sum = 0.f;
  for (int i = threadIdx.x; i < quads; i += blockDim.x) {
    float4 v = x[i];
    if (dl) {
      const float4 d = dl[i];
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      if (store_sum) x[i] = v;
    }
    row4[i] = v;
    sum += (v.x + v.y) + (v.z + v.w);
  }
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float ss = 0.f;
  for (int i = threadIdx.x; i < quads; i += blockDim.x) {
    const float4 v = row4[i];
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    ss += fmaf(a, a, b * b) + fmaf(c, c, d * d);
  }
  const float r = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  TO* o = out + static_cast<size_t>(blockIdx.x) * hidden;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  for (int i = threadIdx.x; i < quads; i += blockDim.x) {
    const float4 v = row4[i], g = w4[i];
    store4(o + 4 * i, (v.x - mean) * r * g.x, (v.y - mean) * r * g.y, (v.z - mean) * r * g.z, (v.w - mean) * r * g.w);
  }
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

// The same for four neighbouring channels a thread (C a multiple of 4, rows on 16-byte boundaries, at most kTapsHeld taps) and
// RUN consecutive rows a CTA: the thread's taps and the RUN + K - 1 rows of h it needs are fetched once, all loads ahead of
// the arithmetic; only a row before its request's first row of the step is fetched apart, from the kept rows.
constexpr int kTapsHeld = 4;
template <typename TO, int RUN>
__global__ void __launch_bounds__(256)
taps_pair_vec_kernel(const float* __restrict__ h, const float* __restrict__ wa, const float* __restrict__ wb,
                     const float* __restrict__ kept, const int* __restrict__ q_start, const int* __restrict__ slots,
                     const int* __restrict__ token_entry, TO* __restrict__ out_a, TO* __restrict__ out_b, int n, int C, int K) {
  pdl_trigger();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  // the taps are weights: fetched before the wait for the kernel ahead
  float ta[4][kTapsHeld], tb[4][kTapsHeld];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int j = 0; j < kTapsHeld; ++j) {
      ta[u][j] = j < K ? wa[static_cast<size_t>(c + u) * K + j] : 0.f;
      tb[u][j] = j < K && wb ? wb[static_cast<size_t>(c + u) * K + j] : 0.f;
    }
  pdl_wait();
  const int t0 = blockIdx.x * RUN;
  int first[RUN];
  const float* st[RUN];
#pragma unroll
  for (int r = 0; r < RUN; ++r) {
    const int e = token_entry[min(t0 + r, n - 1)];
    first[r] = q_start[e];
    st[r] = kept ? kept + static_cast<size_t>(slots[e]) * (K - 1) * C + c : nullptr;
  }
  float4 rows[RUN + kTapsHeld - 1];        // rows[i] is row t0 - (K - 1) + i of h
#pragma unroll
  for (int i = 0; i < RUN + kTapsHeld - 1; ++i) {
    const int row = t0 - (K - 1) + i;
    rows[i] = i < RUN + K - 1 && row >= 0 && row < n ? *reinterpret_cast<const float4*>(h + static_cast<size_t>(row) * C + c)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int r = 0; r < RUN; ++r) {
    const int t = t0 + r;
    if (t >= n) break;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kTapsHeld; ++j) {
      if (j >= K) continue;
      const int src = t - (K - 1) + j;
      v = src >= first[r] ? rows[r + j] : *reinterpret_cast<const float4*>(st[r] + static_cast<size_t>((K - 1) - (first[r] - src)) * C);
      const float in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = fmaf(ta[u][j], in[u], a[u]);
        b[u] = fmaf(tb[u][j], in[u], b[u]);
      }
    }
    // the last row read is the token's own
    store4(out_a + static_cast<size_t>(t) * C + c, v.x + a[0], v.y + a[1], v.z + a[2], v.w + a[3]);
    if (wb) store4(out_b + static_cast<size_t>(t) * C + c, v.x + b[0], v.y + b[1], v.z + b[2], v.w + b[3]);
  }
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

// The same for four neighbouring columns a thread (C a multiple of 4, every array on a 16-byte boundary).
__global__ void __launch_bounds__(256)
scale_sum_average_vec_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ sa,
                             const float* __restrict__ b, const float* __restrict__ sb, float* __restrict__ results,
                             const float* __restrict__ mix, int index, size_t total, int C) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
  float4 v = *reinterpret_cast<const float4*>(x + i);
  const float4 av = *reinterpret_cast<const float4*>(a + i);
  const float4 sav = sa ? *reinterpret_cast<const float4*>(sa + c) : one;
  float4 add = make_float4(sav.x * av.x, sav.y * av.y, sav.z * av.z, sav.w * av.w);
  if (b) {
    const float4 bv = *reinterpret_cast<const float4*>(b + i);
    const float4 sbv = sb ? *reinterpret_cast<const float4*>(sb + c) : one;
    add.x += sbv.x * bv.x; add.y += sbv.y * bv.y; add.z += sbv.z * bv.z; add.w += sbv.w * bv.w;
  }
  v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
  if (mix) {
    *reinterpret_cast<float4*>(results + static_cast<size_t>(index + 1) * total + i) = v;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j <= index; ++j) {
      const float m = mix[j];
      const float4 r = *reinterpret_cast<const float4*>(results + static_cast<size_t>(j) * total + i);
      acc.x = fmaf(m, r.x, acc.x); acc.y = fmaf(m, r.y, acc.y); acc.z = fmaf(m, r.z, acc.z); acc.w = fmaf(m, r.w, acc.w);
    }
    const float m = mix[index + 1];
    v = make_float4(fmaf(m, v.x, acc.x), fmaf(m, v.y, acc.y), fmaf(m, v.z, acc.z), fmaf(m, v.w, acc.w));
  }
  *reinterpret_cast<float4*>(x + i) = v;
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

// The same with the row held in registers between the two passes (16-byte accesses; width a multiple of the vector and at most
// kPolyVectors * 256 vectors): the row is read from memory once.
constexpr int kPolyVectors = 12;
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_vec_kernel(const T* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int width, float eps) {
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const V* row = reinterpret_cast<const V*>(z + static_cast<size_t>(blockIdx.x) * width);
  const int vectors = width / VN;
  V held[kPolyVectors];
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int k = 0; k < kPolyVectors; ++k) {
    const int i = k * 256 + threadIdx.x;
    if (i < vectors) {
      held[k] = row[i];
      float f[VN];
      Vec<T>::unpack(held[k], f);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        const float v2 = f[e] * f[e];
        s1 += v2;
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v2 * f[e], v2 * f[e], s3);
      }
    }
  }
  const float n = static_cast<float>(width);
  const float r1 = rsqrtf(block_sum(s1, scratch) / n + eps);
  const float r2 = rsqrtf(block_sum(s2, scratch) / n + eps);
  const float r3 = rsqrtf(block_sum(s3, scratch) / n + eps);
  const float c0 = coef[0] * r1, c1 = coef[1] * r2, c2 = coef[2] * r3, c3 = coef[3];
  V* o = reinterpret_cast<V*>(out + static_cast<size_t>(blockIdx.x) * width);
#pragma unroll
  for (int k = 0; k < kPolyVectors; ++k) {
    const int i = k * 256 + threadIdx.x;
    if (i < vectors) {
      float f[VN];
      Vec<T>::unpack(held[k], f);
#pragma unroll
      for (int e = 0; e < VN; ++e) f[e] = fmaf(c0, f[e], fmaf(c1, f[e] * f[e], fmaf(c2, f[e] * f[e] * f[e], c3)));
      o[i] = Vec<T>::pack(f);
    }
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

// The same with 16-byte accesses (F a multiple of the vector, arrays on 16-byte boundaries).
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_scaled_vec_kernel(const T* __restrict__ gate_up, const int* __restrict__ pair_row, const float* __restrict__ scale,
                           T* __restrict__ out, int F) {
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  pdl_trigger();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VN;
  if (c >= F) return;
  const size_t r = pair_row ? static_cast<size_t>(pair_row[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  const float s = scale ? scale[blockIdx.x] : 1.f;
  float g[VN], u[VN];
  Vec<T>::unpack(*reinterpret_cast<const V*>(gate_up + r * 2 * F + c), g);
  Vec<T>::unpack(*reinterpret_cast<const V*>(gate_up + r * 2 * F + F + c), u);
#pragma unroll
  for (int e = 0; e < VN; ++e) {
    const float ge = s * g[e];
    g[e] = ge / (1.f + expf(-ge)) * (s * u[e]);
  }
  *reinterpret_cast<V*>(out + r * F + c) = Vec<T>::pack(g);
}

}  // namespace b200

// True when every pointer given (null ones aside) is on a 16-byte boundary.
template <typename... P>
static inline bool aligned16(P... p) { return ((0 | ... | reinterpret_cast<uintptr_t>(p)) & 15) == 0; }

extern "C" int b200_layer_norm(float* resid, const float* delta, const float* w, void* out, const int* rows, int n, int hidden,
                               float eps, int store_sum, int out_dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (hidden <= 0) return B200_ERR_BAD_SIZE;
  const size_t smem = sizeof(float) * hidden;
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  const bool vec = hidden % 4 == 0 && aligned16(resid, delta, w, out);
  B200_DISPATCH_DTYPE(out_dtype, TO, launch(vec ? layer_norm_vec_kernel<TO> : layer_norm_kernel<TO>, dim3(n), dim3(256), smem, stream,
                                            resid, delta, w, static_cast<TO*>(out), rows, hidden, eps, store_sum));
  return launch_status();
}

extern "C" int b200_taps_pair(const float* h, const float* wa, const float* wb, const float* kept, const int* q_start,
                              const int* slots, const int* token_entry, void* out_a, void* out_b, int n, int C, int K,
                              int out_dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (C <= 0 || K <= 0 || (K > 1 && !kept)) return B200_ERR_BAD_SIZE;
  const bool vec = C % 4 == 0 && K <= kTapsHeld && aligned16(h, kept, out_a, out_b);
  const int run = vec && n >= 1024 ? 8 : 1;
  dim3 grid((n + run - 1) / run, vec ? (C / 4 + 255) / 256 : (C + 255) / 256);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(out_dtype, TO, {
    if (vec)
      launch(run == 8 ? taps_pair_vec_kernel<TO, 8> : taps_pair_vec_kernel<TO, 1>, grid, dim3(256), 0, stream, h, wa, wb, kept, q_start,
             slots, token_entry, static_cast<TO*>(out_a), static_cast<TO*>(out_b), n, C, K);
    else
      launch(taps_pair_kernel<TO>, grid, dim3(256), 0, stream, h, wa, wb, kept, q_start, slots, token_entry, static_cast<TO*>(out_a),
             static_cast<TO*>(out_b), C, K);
  });
  return launch_status();
}

extern "C" int b200_scale_sum_average(float* x, const float* a, const float* sa, const float* b, const float* sb, float* results,
                                      const float* mix, int index, int n, int C, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (C <= 0 || index < 0) return B200_ERR_BAD_SIZE;
  const size_t total = static_cast<size_t>(n) * C;
  if (C % 4 == 0 && aligned16(x, a, sa, b, sb, results))
    launch(scale_sum_average_vec_kernel, dim3(static_cast<unsigned>((total / 4 + 255) / 256)), dim3(256), 0, stream, x, a, sa, b, sb,
           results, mix, index, total, C);
  else
    launch(scale_sum_average_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, x, a, sa, b, sb, results,
           mix, index, total, C);
  return launch_status();
}

extern "C" int b200_poly_norm(const void* z, const float* coef, void* out, int n, int width, float eps, int dtype,
                              cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int VN = Vec<T>::n;
    const bool vec = width % VN == 0 && width / VN <= kPolyVectors * 256 && aligned16(z, out);
    launch(vec ? poly_norm_vec_kernel<T> : poly_norm_kernel<T>, dim3(n), dim3(256), 0, stream, static_cast<const T*>(z), coef,
           static_cast<T*>(out), width, eps);
  });
  return launch_status();
}

extern "C" int b200_silu_mul_scaled(const void* gate_up, const int* pair_row, const float* scale, void* out, int rows, int F,
                                    int dtype, cudaStream_t stream) {
  using namespace b200;
  if (rows <= 0) return 0;
  if (F <= 0) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int VN = Vec<T>::n;
    const bool vec = F % VN == 0 && aligned16(gate_up, out);
    dim3 grid(rows, vec ? (F / VN + 255) / 256 : (F + 255) / 256);
    if (grid.y > 65535) return B200_ERR_TOO_LARGE;
    launch(vec ? silu_mul_scaled_vec_kernel<T> : silu_mul_scaled_kernel<T>, grid, dim3(256), 0, stream, static_cast<const T*>(gate_up),
           pair_row, scale, static_cast<T*>(out), F);
  });
  return launch_status();
}
