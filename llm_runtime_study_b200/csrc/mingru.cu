// minGRU: a gated recurrence per channel whose gates read the current token only (Feng, Tung, Ahmed, Bengio, Hajimirsadeghi,
// "Were RNNs All We Needed?").  With the rows of one stacked projection [z | u | g] (biases added by the projection):
//
//   z_t   = sigmoid(zl_t)
//   c_t   = u_t + 1/2 where u_t >= 0, sigmoid(u_t) where u_t < 0        (the candidate, always positive)
//   S_t   = (1 - z_t) S_(t-1) + z_t c_t                                 (S = 0 before the first token)
//   out_t = S_t * silu(g_t)
//
// The state, the gates and the candidate are float32.  One thread per (entry, channel) walks the entry's tokens in order;
// only the multiply-adds form a chain: the loads, sigmoids and candidates of a group of tokens are formed together before
// the chain runs over them.  The order of every sum is the token order, so a state does not depend on how a prompt was cut.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(const T* __restrict__ proj, int ld, int z_off, int u_off, int g_off, T* __restrict__ out, float* __restrict__ state,
                   const int* __restrict__ q_start, const int* __restrict__ slots, int width) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int first = q_start[entry], last = q_start[entry + 1];
  if (last <= first) return;
  float* st = state + static_cast<size_t>(slots[entry]) * width + c;
  float S = *st;
  constexpr int U = 8;
  for (int t0 = first; t0 < last; t0 += U) {
    float a[U], b[U], gate[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const bool live = t0 + j < last;
      const T* row = proj + static_cast<size_t>(live ? t0 + j : first) * ld;
      const float zl = to_float(row[z_off + c]), u = to_float(row[u_off + c]), g = to_float(row[g_off + c]);
      const float z = sigmoid_f(zl);
      const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
      a[j] = live ? 1.f - z : 1.f;
      b[j] = live ? z * cand : 0.f;
      gate[j] = g * sigmoid_f(g);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      S = fmaf(a[j], S, b[j]);
      if (t0 + j < last) out[static_cast<size_t>(t0 + j) * width + c] = from_float<T>(S * gate[j]);
    }
  }
  *st = S;
}

}  // namespace b200

// proj rows [n, ld] in the storage type with the z logits at column z_off, u at u_off, g at g_off (each `width` wide);
// out [n, width] in the storage type; state float32 [slots, width]; q_start [entries + 1]; slots [entries].
extern "C" int b200_mingru_scan(const void* proj, int ld, int z_off, int u_off, int g_off, void* out, float* state, const int* q_start,
                                const int* slots, int n, int entries, int width, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (entries <= 0 || n <= 0) return 0;
  if (width <= 0 || z_off < 0 || u_off < 0 || g_off < 0 || ld < width + max(z_off, max(u_off, g_off))) return B200_ERR_BAD_SIZE;
  dim3 grid((width + 127) / 128, entries);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, launch(mingru_scan_kernel<T>, grid, dim3(128), 0, stream, static_cast<const T*>(proj), ld, z_off, u_off,
                                       g_off, static_cast<T*>(out), state, q_start, slots, width));
  return launch_status();
}
