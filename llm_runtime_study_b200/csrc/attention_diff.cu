// Differential attention over the paged cache: every head holds two score maps (two queries and two keys of d columns
// each, laid out [map 1 | map 2]) over the same values; o = softmax(S1) V - lambda * softmax(S2) V, then o is divided by
// its root mean square over the head's value columns and scaled.  Query head j reads key/value head j / (nq / nkv).
// A token's key row in the pages holds both maps side by side ([pages, nkv, page_size, 2 d]), so one pass over the keys
// and one over the values serve both maps.
//
// Two kernels: the preparation (per-map RMS norm with a weight shared by all heads and maps, rotation of the leading
// columns of every map by the token's position, q written out and k, v into the pages), and the attention on CUDA cores
// in 32-bit arithmetic (one warp per token and head, tiles of 32 keys from the first tile the window touches, so the
// order of every sum depends on the token's own position alone).
#include "common.cuh"

namespace b200 {

constexpr int kPrepWarps = 8;

// W neighbouring values in one access (W = 1 or 4; with 4 the address is a multiple of four values).
template <int W, typename T> __device__ __forceinline__ void load_values(const T* p, float* f);
template <> __device__ __forceinline__ void load_values<1, float>(const float* p, float* f) { f[0] = *p; }
template <> __device__ __forceinline__ void load_values<1, __nv_bfloat16>(const __nv_bfloat16* p, float* f) { f[0] = __bfloat162float(*p); }
template <> __device__ __forceinline__ void load_values<4, float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_values<4, __nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <int W, typename T> __device__ __forceinline__ void store_values(T* p, const float* f);
template <> __device__ __forceinline__ void store_values<1, float>(float* p, const float* f) { *p = f[0]; }
template <> __device__ __forceinline__ void store_values<1, __nv_bfloat16>(__nv_bfloat16* p, const float* f) { *p = __float2bfloat16_rn(f[0]); }
template <> __device__ __forceinline__ void store_values<4, float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store_values<4, __nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  uint2 v;
  *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(f[0], f[1]);
  *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = v;
}

// Row layout [q: nq * maps * d | k: nkv * maps * d | v: nkv * dv].  One warp per (token, head map) of q and k, and per
// value head for the copy of v; a lane moves W neighbouring values at a time.
template <typename T, int W>
__global__ void __launch_bounds__(kPrepWarps * 32)
map_norm_rope_write_kernel(const T* __restrict__ rows, int ld, T* __restrict__ q_out, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, float eps, const float* __restrict__ inv_freq, int rot_dims,
                           const int* __restrict__ positions, const int* __restrict__ token_entry,
                           const int* __restrict__ block_table, int table_stride, int page_size, T* __restrict__ k_pool,
                           T* __restrict__ v_pool, int nq, int nkv, int maps, int d, int dv) {
  extern __shared__ __align__(16) float smem[];      // [rot_dims / 2] cos, [rot_dims / 2] sin, then d floats per warp
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int p = positions[t];
  const int half = inv_freq ? rot_dims / 2 : 0;
  float* cs = smem;
  float* sn = smem + half;
  float* mine = smem + 2 * half + warp * d;
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(static_cast<float>(p) * inv_freq[j], &sn[j], &cs[j]);
  __syncthreads();
  const int page = block_table[static_cast<size_t>(token_entry[t]) * table_stride + p / page_size];
  const int slot = p % page_size;
  const int qm = nq * maps, km = nkv * maps;
  const T* row = rows + static_cast<size_t>(t) * ld;
  for (int u = blockIdx.y * kPrepWarps + warp; u < qm + km + nkv; u += gridDim.y * kPrepWarps) {
    if (u >= qm + km) {                       // a value head: copied as it is
      if (page < 0) continue;                 // a padding row has no pages
      const int g = u - qm - km;
      const T* src = row + static_cast<size_t>(qm + km) * d + static_cast<size_t>(g) * dv;
      T* dst = v_pool + ((static_cast<size_t>(page) * nkv + g) * page_size + slot) * dv;
      for (int i = lane * W; i < dv; i += 32 * W) {
        float f[W];
        load_values<W>(src + i, f);
        store_values<W>(dst + i, f);
      }
      continue;
    }
    const bool is_q = u < qm;
    if (!is_q && page < 0) continue;
    const T* src = row + static_cast<size_t>(u) * d;
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
    for (int i = lane * W; i < d; i += 32 * W) {
      float f[W];
      load_values<W>(src + i, f);
#pragma unroll
      for (int e = 0; e < W; ++e) ss = fmaf(f[e], f[e], ss);
      if constexpr (W == 4) *reinterpret_cast<float4*>(mine + i) = make_float4(f[0], f[1], f[2], f[3]);
      else mine[i] = f[0];
    }
    const float r = w ? rsqrtf(warp_sum(ss) / static_cast<float>(d) + eps) : 1.f;
    __syncwarp();
    T* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(t) * qm + u) * d;
    } else {
      const int kh = (u - qm) / maps, m = (u - qm) % maps;
      dst = k_pool + ((static_cast<size_t>(page) * nkv + kh) * page_size + slot) * (static_cast<size_t>(maps) * d) + static_cast<size_t>(m) * d;
    }
    for (int i0 = lane * W; i0 < d; i0 += 32 * W) {
      float f[W];
      if constexpr (W == 4) {
        // half is a multiple of four here: a chunk lies wholly in the first half, the second half or the tail
        auto four = [](const float* q, float* o) {
          const float4 v = *reinterpret_cast<const float4*>(q);
          o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
        };
        float v[4], g[4] = {1.f, 1.f, 1.f, 1.f};
        four(mine + i0, v);
        if (w) four(w + i0, g);
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = v[e] * (w ? r * g[e] : 1.f);
        if (i0 < 2 * half) {
          const bool first = i0 < half;
          const int other = first ? i0 + half : i0 - half, a = first ? i0 : i0 - half;
          float ov[4], og[4] = {1.f, 1.f, 1.f, 1.f}, c[4], sgn[4];
          four(mine + other, ov);
          if (w) four(w + other, og);
          four(cs + a, c);
          four(sn + a, sgn);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float o = ov[e] * (w ? r * og[e] : 1.f);
            f[e] = first ? f[e] * c[e] - o * sgn[e] : f[e] * c[e] + o * sgn[e];
          }
        }
      } else {
        const int i = i0;
        const float v = mine[i] * (w ? r * w[i] : 1.f);
        float o = v;
        if (i < half) {
          const float other = mine[i + half] * (w ? r * w[i + half] : 1.f);
          o = v * cs[i] - other * sn[i];
        } else if (i < 2 * half) {
          const float other = mine[i - half] * (w ? r * w[i - half] : 1.f);
          o = v * cs[i - half] + other * sn[i - half];
        }
        f[0] = o;
      }
      store_values<W>(dst + i0, f);
    }
    __syncwarp();
  }
}

// q [n, nq, 2, d]; keys [pages, nkv, page_size, 2 d]; values [pages, nkv, page_size, dv]; out [n, nq, dv].
template <typename T, int kMaxChunks>
__global__ void __launch_bounds__(128)
diff_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool, T* __restrict__ out,
                           const int* __restrict__ positions, const int* __restrict__ token_entry,
                           const int* __restrict__ block_table, int table_stride, int page_size, int nq, int nkv, int d, int dv,
                           float scale, int window, float lambda, float out_scale, float eps, int normalise) {
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
  float* qs = smem + warp * 2 * d;
  const T* qrow = q + (static_cast<size_t>(token) * nq + head) * 2 * d;
  for (int i = lane; i < 2 * d; i += 32) qs[i] = to_float(qrow[i]);
  __syncwarp();

  const int w0 = window > 0 ? max(0, p - window + 1) : 0;
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  float acc1[kMaxChunks], acc2[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) acc1[c] = acc2[c] = 0.f;

  constexpr int VN = Vec<T>::n;
  for (int t0 = (w0 / 32) * 32; t0 <= p; t0 += 32) {
    const int t = t0 + lane;
    bool valid = t <= p && t >= w0;
    float s1 = -INFINITY, s2 = -INFINITY;
    const int page = valid ? table[t / page_size] : -1;
    valid = valid && page >= 0;
    if (valid) {
      const T* krow = k_pool + ((static_cast<size_t>(page) * nkv + kvh) * page_size + t % page_size) * 2 * d;
      float dot1 = 0.f, dot2 = 0.f;
      if (d % VN == 0) {
        for (int i = 0; i < d; i += VN) {
          float f[VN], g[VN];
          Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::type*>(krow + i), f);
          Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::type*>(krow + d + i), g);
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            dot1 = fmaf(qs[i + e], f[e], dot1);
            dot2 = fmaf(qs[d + i + e], g[e], dot2);
          }
        }
      } else {
        for (int i = 0; i < d; ++i) {
          dot1 = fmaf(qs[i], to_float(krow[i]), dot1);
          dot2 = fmaf(qs[d + i], to_float(krow[d + i]), dot2);
        }
      }
      s1 = dot1 * scale;
      s2 = dot2 * scale;
    }
    const float mt1 = warp_max(s1), mt2 = warp_max(s2);
    if (mt1 == -INFINITY) continue;          // no key of this tile is visible (both maps see the same keys)
    const float n1 = fmaxf(m1, mt1), n2 = fmaxf(m2, mt2);
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
    const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      acc1[c] *= c1;
      acc2[c] *= c2;
    }
    const int count = min(32, p - t0 + 1);
    for (int j = 0; j < count; ++j) {
      const float a = __shfl_sync(0xffffffffu, p1, j), b = __shfl_sync(0xffffffffu, p2, j);
      const int tj = t0 + j;
      if (tj < w0) continue;
      const int pj = table[tj / page_size];
      if (pj < 0) continue;
      const T* vrow = v_pool + ((static_cast<size_t>(pj) * nkv + kvh) * page_size + tj % page_size) * dv;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) {
          const float v = to_float(vrow[i]);
          acc1[c] = fmaf(a, v, acc1[c]);
          acc2[c] = fmaf(b, v, acc2[c]);
        }
      }
    }
    m1 = n1;
    m2 = n2;
  }
  const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? 1.f / l2 : 0.f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    acc1[c] = acc1[c] * i1 - lambda * (acc2[c] * i2);
    if (lane + 32 * c < dv) ss = fmaf(acc1[c], acc1[c], ss);
  }
  const float r = normalise ? rsqrtf(warp_sum(ss) / static_cast<float>(dv) + eps) * out_scale : out_scale;
  T* orow = out + (static_cast<size_t>(token) * nq + head) * dv;
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) orow[i] = from_float<T>(acc1[c] * r);
  }
}

}  // namespace b200

// rows [n, ld] = [q | k | v]; q_w, k_w: d floats or null (no norm); inv_freq: rot_dims / 2 floats or null (no rotation).
extern "C" int b200_map_norm_rope_write(const void* rows, int ld, void* q_out, const float* q_w, const float* k_w, float eps,
                                        const float* inv_freq, int rot_dims, const int* positions, const int* token_entry,
                                        const int* block_table, int table_stride, int page_size, void* k_pool, void* v_pool,
                                        int n, int nq, int nkv, int maps, int d, int dv, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || maps <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > d)
    return B200_ERR_BAD_SIZE;
  if (ld < (nq + nkv) * maps * d + nkv * dv) return B200_ERR_BAD_SIZE;
  const int half = inv_freq ? rot_dims / 2 : 0;
  const size_t smem = sizeof(float) * (2 * half + kPrepWarps * d);
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  const int units = (nq + nkv) * maps + nkv;
  const int blocks_y = n >= 256 ? 1 : min((units + kPrepWarps - 1) / kPrepWarps, 16);
  // four values an access where every head of every array starts on a multiple of four values and of 16 bytes
  const bool wide = d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && half % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_pool) |
                      reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(q_w) | reinterpret_cast<uintptr_t>(k_w)) & 15) == 0;
  B200_DISPATCH_DTYPE(dtype, T, launch(wide ? map_norm_rope_write_kernel<T, 4> : map_norm_rope_write_kernel<T, 1>, dim3(n, blocks_y),
                                       dim3(kPrepWarps * 32), smem, stream, static_cast<const T*>(rows), ld, static_cast<T*>(q_out), q_w,
                                       k_w, eps, inv_freq, rot_dims, positions, token_entry, block_table, table_stride, page_size,
                                       static_cast<T*>(k_pool), static_cast<T*>(v_pool), nq, nkv, maps, d, dv));
  return launch_status();
}

extern "C" int b200_diff_attention_simt(const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
                                        const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
                                        int nq, int nkv, int d, int dv, float scale, int window, float lambda, float out_scale,
                                        float eps, int normalise, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (d <= 0 || dv <= 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0) return B200_ERR_BAD_SIZE;
  if (dv > 256 || d > 512) return B200_ERR_TOO_LARGE;
  dim3 grid(n, (nq + 3) / 4);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  const size_t smem = static_cast<size_t>(4) * 2 * d * sizeof(float);
#define B200_DIFF_SIMT(CH)                                                                                              \
  B200_DISPATCH_DTYPE(dtype, T,                                                                                          \
      launch(diff_attention_simt_kernel<T, CH>, grid, dim3(128), smem, stream, static_cast<const T*>(q),                 \
             static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), static_cast<T*>(out), positions, token_entry, \
             block_table, table_stride, page_size, nq, nkv, d, dv, scale, window, lambda, out_scale, eps, normalise))
  if (dv <= 64) { B200_DIFF_SIMT(2); }
  else if (dv <= 128) { B200_DIFF_SIMT(4); }
  else { B200_DIFF_SIMT(8); }
#undef B200_DIFF_SIMT
  return launch_status();
}
