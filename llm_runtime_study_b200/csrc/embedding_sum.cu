// An embedding that is a sum of tables and a position vector, written straight into the float32 residual rows:
//
//   x_t = E[token_t] + B[row_t] + pos(p_t)
//
//   row_t  = (token_(t-1) * mul_prev + token_t * mul_cur) mod buckets   (a hashed bigram; 64-bit arithmetic)
//            `buckets` (the table's last row) for a sequence's first token (p_t = 0)
//   pos(p) : column 2i is sin(p * f_i), column 2i + 1 is cos(p * f_i); the f_i are formed by the host in float64
//            and the angle and its sine and cosine are formed in float64 here, so that the vector is the correctly
//            rounded one at every position (a float32 angle at position 10^5 is off by about 10^-2 of a turn's
//            last digits already).
//
// The token before a step's first token of a request is not in the batch: it is kept per request slot (`previous`,
// [slots] int32).  Only the CTA of an entry's first token reads it; the same CTA replaces it, behind a barrier, with the
// entry's last token of this step, so one launch does both.  Either table may be left out (null).
#include "common.cuh"

namespace b200 {

template <typename T>
__global__ void __launch_bounds__(512)
embedding_sum_kernel(const int* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ bigram, float* __restrict__ out,
                     const int* __restrict__ positions, const int* __restrict__ token_entry, const int* __restrict__ q_start,
                     const int* __restrict__ slots, int* __restrict__ previous, const double* __restrict__ freq, int hidden,
                     int vocab, int buckets, long long mul_prev, long long mul_cur, float scale) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  int id = ids[token];
  id = min(max(id, 0), vocab - 1);          // ids are checked by the host; a padding row may carry anything
  const int p = positions[token];
  const T* erow = table + static_cast<size_t>(id) * hidden;
  const T* brow = nullptr;
  if (bigram != nullptr) {
    const int entry = token_entry[token];
    const int first = q_start[entry];
    long long row = buckets;
    if (p > 0) {
      int before = token > first ? ids[token - 1] : previous[slots[entry]];
      before = min(max(before, 0), vocab - 1);
      row = (static_cast<long long>(before) * mul_prev + static_cast<long long>(id) * mul_cur) % buckets;
    }
    brow = bigram + static_cast<size_t>(row) * hidden;
    if (token == first) {                   // every thread of this CTA has read the kept token: now it may be replaced
      __syncthreads();
      if (threadIdx.x == 0) previous[slots[entry]] = ids[q_start[entry + 1] - 1];
    }
  }
  float* dst = out + static_cast<size_t>(token) * hidden;
  for (int pair = threadIdx.x; 2 * pair < hidden; pair += blockDim.x) {
    double s = 0.0, c = 0.0;
    if (freq != nullptr) sincos(static_cast<double>(p) * freq[pair], &s, &c);
    const int c0 = 2 * pair, c1 = c0 + 1;
    float x0 = to_float(erow[c0]) * scale;
    if (brow != nullptr) x0 += to_float(brow[c0]);
    dst[c0] = x0 + static_cast<float>(s);
    if (c1 < hidden) {
      float x1 = to_float(erow[c1]) * scale;
      if (brow != nullptr) x1 += to_float(brow[c1]);
      dst[c1] = x1 + static_cast<float>(c);
    }
  }
}

}  // namespace b200

// ids, positions, token_entry [n]; q_start [entries + 1]; slots [entries]; previous [slots] (null with bigram null);
// table [vocab, hidden] and bigram [buckets + 1, hidden] in the storage type; freq [ceil(hidden / 2)] float64 or null;
// out float32 [n, hidden].
extern "C" int b200_embedding_sum(const int* ids, const void* table, const void* bigram, float* out, const int* positions,
                                  const int* token_entry, const int* q_start, const int* slots, int* previous, const double* freq,
                                  int n, int entries, int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur,
                                  float scale, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (hidden <= 0 || vocab <= 0 || entries <= 0 || (bigram != nullptr && (buckets <= 0 || previous == nullptr))) return B200_ERR_BAD_SIZE;
  const int pairs = (hidden + 1) / 2;
  const int threads = pairs >= 512 ? 512 : (pairs + 31) / 32 * 32;      // a pair of columns a thread and pass
  B200_DISPATCH_DTYPE(dtype, T, launch(embedding_sum_kernel<T>, dim3(n), dim3(threads), 0, stream, ids, static_cast<const T*>(table),
                                       static_cast<const T*>(bigram), out, positions, token_entry, q_start, slots, previous, freq,
                                       hidden, vocab, buckets, mul_prev, mul_cur, scale));
  return launch_status();
}
