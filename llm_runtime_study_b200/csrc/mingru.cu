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
//
// Long portions have a second form in three launches, since a chain of thousands of tokens in one thread leaves most of the
// GPU idle: the recurrence is a composition of affine maps S -> a S + b, which is associative.  (1) every (segment of
// kSegment tokens, channel) forms its segment's map (A, B) from S = 0; (2) every (request, channel) walks its segments'
// maps from the kept state and notes the state at which each segment starts; (3) every (segment, channel) runs the chain
// over its tokens from there and writes the outputs; the thread of a request's last segment keeps the state.  The result
// differs from the one-launch form by rounding only (the state at a segment's start went through the segments' maps).
#include "common.cuh"

namespace b200 {

// The float32 run type forms its sigmoids with the accurate exponential and division; the bfloat16 run type, whose inputs
// carry eight bits, with the fast ones (a few units in the last place of a float32), which are a fifth of the instructions.
template <typename T> __device__ __forceinline__ float sigmoid_of(float x);
template <> __device__ __forceinline__ float sigmoid_of<float>(float x) { return 1.f / (1.f + expf(-x)); }
template <> __device__ __forceinline__ float sigmoid_of<__nv_bfloat16>(float x) { return __frcp_rn(1.f + __expf(-x)); }

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
      const float z = sigmoid_of<T>(zl);
      const float cand = u >= 0.f ? u + 0.5f : sigmoid_of<T>(u);
      a[j] = live ? 1.f - z : 1.f;
      b[j] = live ? z * cand : 0.f;
      gate[j] = g * sigmoid_of<T>(g);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      S = fmaf(a[j], S, b[j]);
      if (t0 + j < last) out[static_cast<size_t>(t0 + j) * width + c] = from_float<T>(S * gate[j]);
    }
  }
  *st = S;
}

constexpr int kSegment = 32;

struct MinGruCell {
  float a, b, gate;
};

template <typename T, bool kGate>
__device__ __forceinline__ MinGruCell mingru_cell(const T* __restrict__ row, int z_off, int u_off, int g_off, int c) {
  const float zl = to_float(row[z_off + c]), u = to_float(row[u_off + c]);
  const float z = sigmoid_of<T>(zl);
  const float cand = u >= 0.f ? u + 0.5f : sigmoid_of<T>(u);
  MinGruCell cell{1.f - z, z * cand, 0.f};
  if (kGate) {
    const float g = to_float(row[g_off + c]);
    cell.gate = g * sigmoid_of<T>(g);
  }
  return cell;
}

// (1) the map of every segment: grid (channel blocks, segments); seg_first / seg_count: the segment's tokens.
template <typename T>
__global__ void __launch_bounds__(128)
mingru_segment_maps_kernel(const T* __restrict__ proj, int ld, int z_off, int u_off, const int* __restrict__ seg_first,
                           const int* __restrict__ seg_count, float* __restrict__ seg_a, float* __restrict__ seg_b, int width) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int first = seg_first[seg], count = seg_count[seg];
  float A = 1.f, B = 0.f;
  constexpr int U = 8;
  for (int t0 = 0; t0 < count; t0 += U) {
    MinGruCell cell[U];
#pragma unroll
    for (int j = 0; j < U; ++j)
      cell[j] = mingru_cell<T, false>(proj + static_cast<size_t>(first + min(t0 + j, count - 1)) * ld, z_off, u_off, 0, c);
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (t0 + j < count) {
        A *= cell[j].a;
        B = fmaf(cell[j].a, B, cell[j].b);
      }
  }
  seg_a[static_cast<size_t>(seg) * width + c] = A;
  seg_b[static_cast<size_t>(seg) * width + c] = B;
}

// (2) the state at which every segment starts: grid (channel blocks, entries); entry_seg [entries + 1]: an entry's segments.
// seg_b is overwritten with that state (seg_a is not needed afterwards).
__global__ void __launch_bounds__(128)
mingru_segment_starts_kernel(const float* __restrict__ seg_a, float* __restrict__ seg_b, const float* __restrict__ state,
                             const int* __restrict__ entry_seg, const int* __restrict__ slots, int width) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  float S = state[static_cast<size_t>(slots[entry]) * width + c];
  constexpr int U = 8;
  const int end = entry_seg[entry + 1];
  for (int s0 = entry_seg[entry]; s0 < end; s0 += U) {
    float a[U], b[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const size_t at = static_cast<size_t>(min(s0 + j, end - 1)) * width + c;
      a[j] = seg_a[at];
      b[j] = seg_b[at];
    }
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (s0 + j < end) {
        seg_b[static_cast<size_t>(s0 + j) * width + c] = S;
        S = fmaf(a[j], S, b[j]);
      }
  }
}

// (3) the chain over every segment from its start state, the outputs, and the state kept by an entry's last segment.
template <typename T>
__global__ void __launch_bounds__(128)
mingru_segment_outputs_kernel(const T* __restrict__ proj, int ld, int z_off, int u_off, int g_off, T* __restrict__ out,
                              float* __restrict__ state, const float* __restrict__ seg_start, const int* __restrict__ seg_first,
                              const int* __restrict__ seg_count, const int* __restrict__ seg_slot, int width) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int first = seg_first[seg], count = seg_count[seg];
  float S = seg_start[static_cast<size_t>(seg) * width + c];
  constexpr int U = 8;
  for (int t0 = 0; t0 < count; t0 += U) {
    MinGruCell cell[U];
#pragma unroll
    for (int j = 0; j < U; ++j)
      cell[j] = mingru_cell<T, true>(proj + static_cast<size_t>(first + min(t0 + j, count - 1)) * ld, z_off, u_off, g_off, c);
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (t0 + j < count) {
        S = fmaf(cell[j].a, S, cell[j].b);
        out[static_cast<size_t>(first + t0 + j) * width + c] = from_float<T>(S * cell[j].gate);
      }
  }
  const int slot = seg_slot[seg];       // -1 unless the segment is its entry's last
  if (slot >= 0) state[static_cast<size_t>(slot) * width + c] = S;
}

}  // namespace b200

extern "C" int b200_mingru_segment_tokens() { return b200::kSegment; }

// The three-launch form.  The caller cuts every entry into segments of at most b200_mingru_segment_tokens() tokens:
// seg_first, seg_count, seg_slot [segments] (seg_slot: the entry's slot for its last segment, else -1), entry_seg
// [entries + 1] (the entry's first segment; segments of an entry follow one another in token order).  scratch: float32
// [2, segments, width].
extern "C" int b200_mingru_scan_segments(const void* proj, int ld, int z_off, int u_off, int g_off, void* out, float* state,
                                         const int* slots, const int* seg_first, const int* seg_count, const int* seg_slot,
                                         const int* entry_seg, float* scratch, int n, int entries, int segments, int width, int dtype,
                                         cudaStream_t stream) {
  using namespace b200;
  if (entries <= 0 || n <= 0 || segments <= 0) return 0;
  if (width <= 0 || z_off < 0 || u_off < 0 || g_off < 0 || ld < width + max(z_off, max(u_off, g_off))) return B200_ERR_BAD_SIZE;
  dim3 per_segment((width + 127) / 128, segments), per_entry((width + 127) / 128, entries);
  if (per_segment.y > 65535 || per_entry.y > 65535) return B200_ERR_TOO_LARGE;
  float* seg_a = scratch;
  float* seg_b = scratch + static_cast<size_t>(segments) * width;
  B200_DISPATCH_DTYPE(dtype, T, {
    launch(mingru_segment_maps_kernel<T>, per_segment, dim3(128), 0, stream, static_cast<const T*>(proj), ld, z_off, u_off, seg_first,
           seg_count, seg_a, seg_b, width);
    launch(mingru_segment_starts_kernel, per_entry, dim3(128), 0, stream, seg_a, seg_b, state, entry_seg, slots, width);
    launch(mingru_segment_outputs_kernel<T>, per_segment, dim3(128), 0, stream, static_cast<const T*>(proj), ld, z_off, u_off, g_off,
           static_cast<T*>(out), state, seg_b, seg_first, seg_count, seg_slot, width);
  });
  return launch_status();
}

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
