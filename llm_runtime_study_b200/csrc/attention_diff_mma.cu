// bfloat16 tensor-core differential attention over the paged cache, built once per pair of sizes
// (-DDIFF_DIM=<columns of one map of q and k> -DDIFF_VDIM=<value columns>, both multiples of 16).
//
// Every head has two score maps over the same values: o = softmax(S1) V - lambda softmax(S2) V, then o is divided by its
// root mean square over the value columns and scaled.  A token's key row holds both maps side by side (2 d columns).
//
// A CTA takes up to BM = 64 rows: consecutive query tokens of one request times the query heads that share one key/value
// head (at most 64 of them a CTA).  Keys and values are streamed in tiles of 32 tokens through shared memory (cp.async,
// two stages, three for single tokens) from the request's pages.  Eight warps: warp w owns rows 16 (w & 3) .. + 15 of
// map (w >> 2): it forms
// S = Q_m K_m^T (mma.sync m16n8k16, float accumulation), runs the online softmax in float32, rounds P to bfloat16 and
// multiplies it with all value columns.  At the end the warps of map 2 hand their normalised rows to the warps of map 1
// through shared memory, which subtract, normalise and store.  Single tokens may have their keys cut into parts: every
// part leaves (maximum, sum, unnormalised output) per row and map in scratch memory and a second launch merges the parts
// of both maps and finishes the row.  A single token whose heads fit 16 rows runs the second form of the kernel: the
// four warps of a map all form the same S for rows 0 .. 15 and each multiplies P with its own quarter of the value
// columns, so that every warp works and a thread holds a quarter of the accumulators (two CTAs a multiprocessor).
// Key t is visible to a query at position p iff t <= p and (window == 0 or t > p - window).
#include "common.cuh"
#include "mma.cuh"

#if !defined(DIFF_DIM) || !defined(DIFF_VDIM)
#error "compile with -DDIFF_DIM=<columns of one map> -DDIFF_VDIM=<value columns>"
#endif
static_assert(DIFF_DIM % 16 == 0 && DIFF_DIM >= 16 && DIFF_DIM <= 256, "a map's width must be 16..256 in steps of 16");
static_assert(DIFF_VDIM % 16 == 0 && DIFF_VDIM >= 16 && DIFF_VDIM <= 256, "the value width must be 16..256 in steps of 16");

namespace b200 {

using bf16 = __nv_bfloat16;
constexpr int D = DIFF_DIM, DK = 2 * DIFF_DIM, DV = DIFF_VDIM;
constexpr int BM = 64, BN = 32, NT = 256;
constexpr int LDK = DK + 8;                 // padded rows: ldmatrix rows fall into different banks
constexpr int LDV = DV + 8;
constexpr int KSTEPS = D / 16;
constexpr int OTILES = DV / 8;
constexpr int kStreamBytes = ((BM + 2 * BN) * LDK + 2 * BN * LDV) * 2;
constexpr int kExchangeBytes = BM * DV * 4;  // the rows of map 2, float32, after the last tile
constexpr int kSmemBytes = kStreamBytes > kExchangeBytes ? kStreamBytes : kExchangeBytes;
// the value columns of a single token's rows are shared out over a map's warps, an even number of 8-column tiles each
constexpr int kColParts = OTILES % 8 == 0 ? 4 : OTILES % 4 == 0 ? 2 : 1;
constexpr int kSingleRows = 16;
constexpr int kSingleStages = 3;                          // its tiles are short of work, so more of them are in flight
constexpr int kSingleSmemBytes = ((kSingleRows + kSingleStages * BN) * LDK + kSingleStages * BN * LDV) * 2;

struct DiffParams {
  const bf16* q;            // [n, nq, 2 D]
  const bf16* k_pool;       // [pages, nkv, page_size, 2 D]
  const bf16* v_pool;       // [pages, nkv, page_size, DV]
  bf16* out;                // [n, nq, DV]
  const int* positions;     // [n]
  const int* block_table;   // [entries, table_stride]
  const int* tile_entry;    // per tile: entry, first token (index into the batch's rows), tokens
  const int* tile_start;
  const int* tile_count;
  int table_stride, page_size, nq, nkv, group, group_heads, slices, tokens_per_tile, window;
  float scale_log2, lambda, out_scale, eps;
  int normalise;
  // a tile's keys cut into `splits` parts (single tokens only): CTA z takes its share of the key tiles and leaves
  // (maximum, sum) and the unnormalised output of row (token * nq + head) * 2 + map in scratch memory
  int splits;
  int merge;        // parts are left in scratch memory (also with one part) and a second launch finishes the rows
  float* part_o;    // [rows][splits][DV]
  float* part_ml;   // [rows][splits][2]
};

// Eight threads a row: the page of the row is looked up once and each thread copies every eighth 16-byte piece of the key row
// and of the value row.
static_assert(NT / 8 == BN, "a tile's rows are shared out eight threads each");
__device__ __forceinline__ void load_tiles(bf16* ks, bf16* vs, const DiffParams& p, const int* table, int kvh, int t0, int lo, int hi) {
  constexpr int CK = DK / 8, CV = DV / 8;
  const int r = threadIdx.x >> 3, piece = threadIdx.x & 7;
  const int t = t0 + r;
  const bf16* ksrc = p.k_pool;
  const bf16* vsrc = p.v_pool;
  int bytes = 0;
  if (t >= lo && t <= hi) {
    const int index = t / p.page_size;
    const int page = table[index];
    if (page >= 0) {
      const size_t row = (static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + (t - index * p.page_size);
      ksrc += row * DK;
      vsrc += row * DV;
      bytes = 16;
    }
  }
  const int step = bytes ? 8 : 0;          // a row that is not copied (zeros are written) reads no address but the pool's first
#pragma unroll
  for (int ch = piece; ch < CK; ch += 8) cp_async_16(ks + r * LDK + ch * 8, ksrc + ch * step, bytes);
#pragma unroll
  for (int ch = piece; ch < CV; ch += 8) cp_async_16(vs + r * LDV + ch * 8, vsrc + ch * step, bytes);
}

// kSingle: every tile is one token whose heads of a key/value head fit kSingleRows rows; parts go to scratch memory.
template <bool kSingle>
__global__ void __launch_bounds__(NT, kSingle ? 2 : 1)
diff_attention_mma_kernel(const DiffParams p) {
  constexpr int QROWS = kSingle ? kSingleRows : BM;
  constexpr int STAGES = kSingle ? kSingleStages : 2;
  constexpr int OT = kSingle ? OTILES / kColParts : OTILES;       // the output tiles of 8 columns a warp owns
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* ks = qs + QROWS * LDK;
  bf16* vs = ks + STAGES * BN * LDK;
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x;
  const int kvh = blockIdx.y / p.slices, slice = blockIdx.y - kvh * p.slices;
  const int entry = p.tile_entry[tile], start = p.tile_start[tile], count = p.tile_count[tile];
  const int hg = min(p.group_heads, p.group - slice * p.group_heads);
  const int head0 = kvh * p.group + slice * p.group_heads;
  const int* table = p.block_table + static_cast<size_t>(entry) * p.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int map = warp >> 2;
  const int rg = kSingle ? 0 : (warp & 3);                        // the warp's 16 rows
  const int col0 = kSingle ? (warp & 3) * OT * 8 : 0;             // its first value column

  // the rows of this thread: r0 = 16 rg + lane / 4 and r0 + 8; row r is token r / hg, head r % hg of the tile
  int pos[2], row_token[2], row_head[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rg * 16 + (lane >> 2) + i * 8;
    const int tl = r / hg, hl = r - tl * hg;
    const bool valid = tl < count && tl < p.tokens_per_tile;
    row_token[i] = valid ? start + tl : -1;
    row_head[i] = head0 + hl;
    pos[i] = valid ? p.positions[start + tl] : -1;
  }
  const int p_first = p.positions[start], p_last = p.positions[start + count - 1];
  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0, hi = p_last;

  // Q tile: both maps of every row
  {
    constexpr int CH = DK / 8;
    for (int c = threadIdx.x; c < QROWS * CH; c += NT) {
      const int r = c / CH, ch = c - r * CH;
      const int tl = r / hg, hl = r - tl * hg;
      const bool valid = tl < count && tl < p.tokens_per_tile;
      const bf16* src = valid ? p.q + (static_cast<size_t>(start + tl) * p.nq + head0 + hl) * DK + ch * 8 : p.q;
      cp_async_16(qs + r * LDK + ch * 8, src, valid ? 16 : 0);
    }
  }
  int t_begin = (lo / BN) * BN;
  int tiles = hi >= t_begin ? (hi - t_begin) / BN + 1 : 0;
  if (p.splits > 1) {          // this CTA's share of the key tiles
    const int per = (tiles + p.splits - 1) / p.splits;
    const int first_tile = min(tiles, static_cast<int>(blockIdx.z) * per);
    tiles = min(tiles - first_tile, per);
    t_begin += first_tile * BN;
  }
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {        // one group a stage, empty ones too: the waits count groups
    if (st < tiles) load_tiles(ks + st * BN * LDK, vs + st * BN * LDV, p, table, kvh, t_begin + st * BN, lo, hi);
    cp_async_commit();
  }

  float o[OT][4];
#pragma unroll
  for (int j = 0; j < OT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  // a warp none of whose rows is a (token, head) of the tile only helps with the copies
  const bool warp_live = kSingle ? (warp & 3) < kColParts : (rg * 16) / hg < min(count, p.tokens_per_tile);

  for (int kt = 0; kt < tiles; ++kt) {
    const int t0 = t_begin + kt * BN;
    const bf16* kcur = ks + (kt % STAGES) * BN * LDK;
    const bf16* vcur = vs + (kt % STAGES) * BN * LDV;
    if (kt + STAGES - 1 < tiles) {
      const int st = (kt + STAGES - 1) % STAGES;
      load_tiles(ks + st * BN * LDK, vs + st * BN * LDV, p, table, kvh, t0 + (STAGES - 1) * BN, lo, hi);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (!warp_live) {
      __syncthreads();
      continue;
    }
    // S = Q_m K_m^T for this warp's 16 rows and the tile's 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4], b[2][4];
      ldmatrix_x4(a, qs + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + map * D + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        ldmatrix_x4(b[j], kcur + (j * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + map * D + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) mma_bf16(s[j], a, b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
    // mask, online softmax (base 2)
    float m_new[2] = {m[0], m[1]};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int t = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = pos[i] >= 0 && t <= pos[i] && (p.window == 0 || t > pos[i] - p.window);
        s[j][e] = seen ? s[j][e] * p.scale_log2 : -INFINITY;
        m_new[i] = fmaxf(m_new[i], s[j][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
    }
    float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float base = m_new[i] == -INFINITY ? 0.f : m_new[i];
      corr[i] = exp2f(m[i] - base);        // m = -inf: 0
      m[i] = m_new[i];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s[j][i * 2 + e] - base);
          s[j][i * 2 + e] = pv;
          sum[i] += pv;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      l[i] = l[i] * corr[i] + sum[i];
    }
#pragma unroll
    for (int j = 0; j < OT; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < OT; j += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vcur + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + col0 + j * 8 + (lane >> 4) * 8);
        mma_bf16(o[j], a, b[0], b[1]);
        mma_bf16(o[j + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (kSingle || p.merge) {
    if (!warp_live) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (row_token[i] < 0) continue;
      const size_t slot = ((static_cast<size_t>(row_token[i]) * p.nq + row_head[i]) * 2 + map) * p.splits + blockIdx.z;
      if ((lane & 3) == 0 && col0 == 0) {
        p.part_ml[slot * 2] = m[i];
        p.part_ml[slot * 2 + 1] = l[i];
      }
      float* dst = p.part_o + slot * DV + col0 + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < OT; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][i * 2], o[j][i * 2 + 1]);
    }
    return;
  }
  if constexpr (!kSingle) {
  // map 2's rows through shared memory (the tiles are done with: every warp passed the loop's last barrier)
  float* xs = reinterpret_cast<float*>(smem_raw);
  __syncthreads();
  if (map == 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
      float* dst = xs + (rg * 16 + (lane >> 2) + i * 8) * DV + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < OTILES; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
    }
  }
  __syncthreads();
  if (map == 1) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    const float* other = xs + (rg * 16 + (lane >> 2) + i * 8) * DV + (lane & 3) * 2;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < OTILES; ++j) {
      const float2 b = *reinterpret_cast<const float2*>(other + j * 8);
      const float x = o[j][i * 2] * inv - p.lambda * b.x, y = o[j][i * 2 + 1] * inv - p.lambda * b.y;
      o[j][i * 2] = x;
      o[j][i * 2 + 1] = y;
      ss = fmaf(x, x, fmaf(y, y, ss));
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (row_token[i] < 0) continue;
    const float r = p.normalise ? rsqrtf(ss / static_cast<float>(DV) + p.eps) * p.out_scale : p.out_scale;
    bf16* dst = p.out + (static_cast<size_t>(row_token[i]) * p.nq + row_head[i]) * DV + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < OTILES; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][i * 2] * r, o[j][i * 2 + 1] * r);
  }
  }
}

// A row's parts merged per map (a_m = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z, M the largest maximum), then
// o = a_1 - lambda a_2, its root mean square over the value columns, the scale.  The parts' factors are formed once, in
// shared memory, from one load a part; the sums over the parts then run over loads that do not wait for one another.
constexpr int kMaxSplits = 64;
__global__ void __launch_bounds__(128)
diff_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out, int splits, float lambda,
                  float out_scale, float eps, int normalise) {
  __shared__ float warp_ss[4];
  __shared__ float part_m[2][kMaxSplits], part_l[2][kMaxSplits], factor[2][kMaxSplits];
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  if (threadIdx.x < 2 * splits) {
    const int mp = threadIdx.x / splits, z = threadIdx.x - mp * splits;
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((row * 2 + mp) * splits + z) * 2);
    part_m[mp][z] = ml.x;
    part_l[mp][z] = ml.y;
  }
  __syncthreads();
  if (threadIdx.x < 2) {            // one thread a map, the parts in their order
    const int mp = threadIdx.x;
    float t = -INFINITY;
    for (int z = 0; z < splits; ++z) t = fmaxf(t, part_m[mp][z]);
    float total = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float f = part_m[mp][z] == -INFINITY ? 0.f : exp2f(part_m[mp][z] - t);
      factor[mp][z] = f;
      total += f * part_l[mp][z];
    }
    const float inv = total > 0.f ? 1.f / total : 0.f;
    for (int z = 0; z < splits; ++z) factor[mp][z] *= inv;
  }
  __syncthreads();
  constexpr int PER = (DV + 127) / 128;
  float vals[PER];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const int c = threadIdx.x + u * 128;
    vals[u] = 0.f;
    if (c >= DV) continue;
    float a[2];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      const float* po = part_o + (row * 2 + mp) * splits * DV + c;
      float acc = 0.f;
#pragma unroll 8
      for (int z = 0; z < splits; ++z) acc = fmaf(factor[mp][z], po[static_cast<size_t>(z) * DV], acc);   // a part without keys left zeros
      a[mp] = acc;
    }
    vals[u] = a[0] - lambda * a[1];
    ss = fmaf(vals[u], vals[u], ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = (warp_ss[0] + warp_ss[1]) + (warp_ss[2] + warp_ss[3]);
  const float r = normalise ? rsqrtf(ss / static_cast<float>(DV) + eps) * out_scale : out_scale;
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const int c = threadIdx.x + u * 128;
    if (c < DV) out[row * DV + c] = __float2bfloat16_rn(vals[u] * r);
  }
}

DeviceOnce diff_once, diff_single_once;

}  // namespace b200

extern "C" int b200_attention_diff_dim() { return b200::D; }
extern "C" int b200_attention_diff_vdim() { return b200::DV; }

// q [n, nq, 2 D], keys [pages, nkv, page_size, 2 D], values [pages, nkv, page_size, DV], out [n, nq, DV]; tiles: (entry, first
// row, rows) of consecutive tokens of one entry, at most max(1, 64 / min(64, nq / nkv)) each.  With scratch memory (every tile is
// token t alone, tile t): the keys of a token are cut into `splits` parts (one or more), merged by a second launch; scratch holds
// 2 * splits * (DV + 2) floats per (token, head).
extern "C" int b200_attention_diff_bf16(const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
                                        const int* block_table, int table_stride, int page_size, int nq, int nkv, float scale, int window,
                                        float lambda, float out_scale, float eps, int normalise, const int* tile_entry,
                                        const int* tile_start, const int* tile_count, int num_tiles, int splits, float* scratch,
                                        long scratch_floats, cudaStream_t stream) {
  using namespace b200;
  if (num_tiles <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || window < 0 || splits < 1 || splits > kMaxSplits) return B200_ERR_BAD_SIZE;
  const bool merge = splits > 1 || scratch != nullptr;
  if (merge && (scratch == nullptr || scratch_floats < static_cast<long>(num_tiles) * nq * 2 * splits * (DV + 2))) return 10004;
  const bool single = merge && nq / nkv <= kSingleRows;
  const int status = single ? configure_once(diff_single_once, diff_attention_mma_kernel<true>, kSingleSmemBytes)
                            : configure_once(diff_once, diff_attention_mma_kernel<false>, kSmemBytes);
  if (status != 0) return status;
  DiffParams p{};
  p.q = static_cast<const bf16*>(q);
  p.k_pool = static_cast<const bf16*>(k_pool);
  p.v_pool = static_cast<const bf16*>(v_pool);
  p.out = static_cast<bf16*>(out);
  p.positions = positions;
  p.block_table = block_table;
  p.tile_entry = tile_entry;
  p.tile_start = tile_start;
  p.tile_count = tile_count;
  p.table_stride = table_stride;
  p.page_size = page_size;
  p.nq = nq;
  p.nkv = nkv;
  p.group = nq / nkv;
  p.group_heads = p.group < BM ? p.group : BM;
  p.slices = (p.group + p.group_heads - 1) / p.group_heads;
  p.tokens_per_tile = BM / p.group_heads;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lambda = lambda;
  p.out_scale = out_scale;
  p.eps = eps;
  p.normalise = normalise;
  p.splits = splits;
  p.merge = merge ? 1 : 0;
  if (merge) {
    p.tokens_per_tile = 1;
    p.part_o = scratch;
    p.part_ml = scratch + static_cast<size_t>(num_tiles) * nq * 2 * splits * DV;
  }
  dim3 grid(num_tiles, nkv * p.slices, splits);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  if (single)
    launch(diff_attention_mma_kernel<true>, grid, dim3(NT), kSingleSmemBytes, stream, p);
  else
    launch(diff_attention_mma_kernel<false>, grid, dim3(NT), kSmemBytes, stream, p);
  if (merge)
    launch(diff_merge_kernel, dim3(num_tiles * nq), dim3(128), 0, stream, p.part_o, p.part_ml, p.out, splits, lambda, out_scale, eps, normalise);
  return launch_status();
}
