// Expert-parallel step over peer memory: the route plan and the quantize-and-send kernel.
//
// Rank r of G owns experts [r*L, (r+1)*L).  After the ranks have gathered each other's
// per-expert row counts (one small collective), every rank can compute on its own device
// where each of its rows lands on the owner and where each row it computes has to go back:
// no row count ever travels to the host.  The quantizer then writes packed rows straight into
// the owners' GEMM operand buffers through peer pointers (plain stores over NVLink), and the
// fc2 GEMM writes its BF16 rows straight into the source ranks' buffers through the per-row
// pointer table built here.  Scale factors travel row-major (32 contiguous bytes per warp
// store: the 4-byte pieces of the swizzled atoms cost three times as long on the link) and
// the owner swizzles them into atoms with a local kernel.
//
// Row order on the owner: expert-major, within an expert by source rank, within a source in
// the source's own (stable) expert-major order.
#include "common.cuh"
#include "quantize_math.cuh"

namespace lm {
namespace {

// status word of this file's kernels (read and cleared together with the GEMM's)
__device__ uint32_t g_ep_status = 0;

constexpr int kMaxRanks = LM_EP_MAX_RANKS;
constexpr int kMaxExperts = 256;
constexpr int kPlanThreads = 256;
constexpr int kPlanTileRows = 128;

struct PlanParams {
  const int32_t* counts_all;  // [world, experts]: row g = rows rank g holds for every expert
  int world;
  int rank;
  int experts;
  int local_experts;
  int64_t max_rows;       // rows the owners' operand buffers hold
  int64_t row_bytes;      // bytes of one returned row
  uint64_t return_base[kMaxRanks];  // address of every rank's return buffer
  int32_t* own_indptr;    // [local_experts + 1] expert bounds of the rows this rank receives
  int32_t* dest_base;     // [experts] owner row where this rank's rows of expert e begin
  int32_t* owner_start;   // [experts] owner row where expert e begins
  uint64_t* row_ptrs;     // [max_rows] where each received row's result goes
  int32_t* out_blocks;    // optional [(max_rows/128 + local_experts) * 4][2]: per 32-row block of a
                          // 128-row tile (atom row of its scale factors, quarter) the source rank and
                          // the first row in that rank's return buffer, or -1 when the block is not
                          // 32 whole rows of one (expert, source) segment
  int32_t* valid;         // 1 when every owner's rows fit max_rows
};

// Every CTA rebuilds the (tiny) plan in shared memory; CTA 0 writes the tables, and the
// CTAs share the (expert, source) segments of the row-pointer table.
__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(PlanParams p) {
  __shared__ int s_cnt[kMaxRanks][kMaxExperts];
  __shared__ int s_src_start[kMaxRanks][kMaxExperts];  // source g's own m_indptr
  __shared__ int s_owner_start[kMaxExperts];
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_owner_rows[kMaxRanks];
  const int tid = threadIdx.x;
  const int E = p.experts, G = p.world, L = p.local_experts;
  for (int i = tid; i < G * E; i += kPlanThreads) s_cnt[i / E][i % E] = __ldg(p.counts_all + i);
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += kPlanThreads) {
    int total = 0;
    for (int g = 0; g < G; ++g) total += s_cnt[g][e];
    s_total[e] = total;
  }
  __syncthreads();
  // Warp w: exclusive prefix over the experts of source w, then over the local experts of
  // owner w.  A lane owns a run of consecutive entries; a warp scan joins the runs.
  for (int g = warp; g < G; g += kPlanThreads / 32) {
    const int per_lane = (E + 31) / 32;
    int sum = 0;
    for (int i = 0; i < per_lane; ++i) {
      const int e = lane * per_lane + i;
      if (e < E) sum += s_cnt[g][e];
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += up;
    }
    int run = incl - sum;
    for (int i = 0; i < per_lane; ++i) {
      const int e = lane * per_lane + i;
      if (e < E) {
        s_src_start[g][e] = run;
        run += s_cnt[g][e];
      }
    }
    // owner g
    const int per_lane_l = (L + 31) / 32;
    sum = 0;
    for (int i = 0; i < per_lane_l; ++i) {
      const int l = lane * per_lane_l + i;
      if (l < L) sum += s_total[g * L + l];
    }
    incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += up;
    }
    run = incl - sum;
    for (int i = 0; i < per_lane_l; ++i) {
      const int l = lane * per_lane_l + i;
      if (l < L) {
        s_owner_start[g * L + l] = run;
        run += s_total[g * L + l];
      }
    }
    if (lane == 31) s_owner_rows[g] = incl;
  }
  __syncthreads();
  bool fits = true;
  for (int g = 0; g < G; ++g) fits = fits && s_owner_rows[g] <= p.max_rows;

  if (blockIdx.x == 0) {
    for (int e = tid; e < E; e += kPlanThreads) {
      int before = 0;
      for (int g = 0; g < p.rank; ++g) before += s_cnt[g][e];
      p.dest_base[e] = s_owner_start[e] + before;
      p.owner_start[e] = s_owner_start[e];
    }
    // an oversized step computes nothing: empty experts, and the flag for the host
    for (int l = tid; l <= L; l += kPlanThreads)
      p.own_indptr[l] = !fits ? 0 : (l < L ? s_owner_start[p.rank * L + l] : s_owner_rows[p.rank]);
    if (tid == 0) {
      *p.valid = fits ? 1 : 0;
      if (!fits) atomicOr(&g_ep_status, static_cast<uint32_t>(LM_STATUS_EP_OVERFLOW));
    }
  }
  if (!fits) return;
  for (int seg = blockIdx.x; seg < L * G; seg += gridDim.x) {
    const int l = seg / G, g = seg % G;
    const int e = p.rank * L + l;
    int before = 0;
    for (int h = 0; h < g; ++h) before += s_cnt[h][e];
    const int first = s_owner_start[e] + before;
    const int64_t src_row = s_src_start[g][e];
    const int rows = s_cnt[g][e];
    for (int i = tid; i < rows; i += kPlanThreads)
      p.row_ptrs[first + i] = p.return_base[g] + static_cast<uint64_t>(src_row + i) * p.row_bytes;
  }
  if (p.out_blocks == nullptr) return;
  // 32-row blocks that lie inside one segment leave the fc2 kernel as one bulk store each: the
  // rows of a segment are consecutive in the source's return buffer
  for (int l = blockIdx.x; l < L; l += gridDim.x) {
    const int e = p.rank * L + l;
    const int begin = s_owner_start[e];
    const int total = s_total[e];
    const int first_tile = begin / kPlanTileRows + l;
    const int blocks = ((total + kPlanTileRows - 1) / kPlanTileRows) * 4;
    for (int b = tid; b < blocks; b += kPlanThreads) {
      const int lo = b * 32;  // first row of the block, counted from the expert's first row
      int rank = -1, ret_row = 0;
      if (lo + 32 <= total) {
        int seg_lo = 0;
        for (int g = 0; g < G; ++g) {
          const int seg_hi = seg_lo + s_cnt[g][e];
          if (lo >= seg_lo && lo + 32 <= seg_hi) {
            rank = g;
            ret_row = s_src_start[g][e] + (lo - seg_lo);
            break;
          }
          seg_lo = seg_hi;
        }
      }
      p.out_blocks[2 * (first_tile * 4 + b)] = rank;
      p.out_blocks[2 * (first_tile * 4 + b) + 1] = ret_row;
    }
  }
}

// ------------------------------------------------ quantize once, send to the owners
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTileRows = 128;
constexpr int kTileCols = 512;  // 32 lanes x 16 elements

struct SendParams {
  const __nv_bfloat16* x;
  int64_t tokens;
  int features;
  int top_k;
  int local_experts;
  const int32_t* slots;        // (tokens*top_k) row in this rank's expert-major order, -1 = dropped
  const int32_t* topk_ids;     // global expert ids
  const int32_t* src_indptr;   // this rank's dispatch bounds over the global experts
  const int32_t* dest_base;
  const int32_t* owner_start;
  const int32_t* valid;
  const float* scale_pair;
  uint8_t* q[kMaxRanks];       // every rank's packed-row buffer
  uint8_t* sf[kMaxRanks];      // every rank's row-major scale factors, features/16 bytes a row
};

// One warp per token, as in the single-GPU scatter quantizer; only the destinations differ:
// the owner's buffers and the rows the route plan assigns.
__global__ void __launch_bounds__(kThreads) ep_quantize_send_kernel(SendParams p) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (token >= p.tokens || __ldg(p.valid) == 0) return;
  uint8_t* my_q = nullptr;
  uint8_t* my_sf = nullptr;
  if (lane < p.top_k) {
    const int slot = __ldg(p.slots + token * p.top_k + lane);
    if (slot >= 0) {
      const int e = __ldg(p.topk_ids + token * p.top_k + lane);
      const int owner = e / p.local_experts;
      const int64_t row = __ldg(p.dest_base + e) + (slot - __ldg(p.src_indptr + e));
      my_q = p.q[owner] + row * (p.features >> 1);
      my_sf = p.sf[owner] + row * (p.features >> 4);
    }
  }
  const float pts = __ldg(p.scale_pair);
  const float inv_pts = __ldg(p.scale_pair + 1);
  const __nv_bfloat16* x_row = p.x + token * p.features;
  Slice<__nv_bfloat16> cur, next;
  int col = lane * 16;
  if (col < p.features) cur.load(x_row + col);
  for (; col - lane * 16 < p.features; col += kTileCols) {
    const bool col_ok = col < p.features;
    const int next_col = col + kTileCols;
    if (next_col < p.features) next.load(x_row + next_col);
    uint2 packed = make_uint2(0, 0);
    uint32_t sf_byte = 0;
    if (col_ok) sf_byte = quantize_group(cur, pts, inv_pts, true, &packed);
    uint32_t word = sf_byte;
    word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 1) << 8;
    word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 2) << 16;
    word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 3) << 24;
    for (int j = 0; j < p.top_k; ++j) {
      uint8_t* q_row = reinterpret_cast<uint8_t*>(
          __shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(my_q), j));
      uint8_t* sf_row = reinterpret_cast<uint8_t*>(
          __shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(my_sf), j));
      if (q_row == nullptr || !col_ok) continue;
      *reinterpret_cast<uint2*>(q_row + (col >> 1)) = packed;
      if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(sf_row + (col >> 4)) = word;
    }
    cur = next;
  }
}

// ------------------------------------------------ row-major scale factors -> atoms
// One CTA per (128-row scale-factor tile, 2048-feature slice): the tile's rows are read
// whole (coalesced) into shared memory and leave as 16-byte pieces of the 512-byte atoms,
// piece (r % 32) of an atom holding the four factors of rows r, r+32, r+64, r+96.
constexpr int kSwizzleCols = 128;  // scale-factor bytes of a row handled per CTA (2048 features)

struct SwizzleParams {
  const uint8_t* linear;   // (rows, features/16)
  const int32_t* m_indptr;
  int experts;
  int features;
  uint8_t* atoms;          // varlen atoms: expert e starts at atom row m_indptr[e]/128 + e
};

__global__ void __launch_bounds__(kThreads) ep_sf_swizzle_kernel(SwizzleParams p) {
  __shared__ __align__(16) uint8_t s_rows[kTileRows][kSwizzleCols + 16];  // padded against bank conflicts
  __shared__ int s_tile[3];  // first row, valid rows, found
  const int tid = threadIdx.x;
  if (tid == 0) s_tile[2] = 0;
  __syncthreads();
  // thread e checks whether expert e's atom rows contain this CTA's (at most one does)
  for (int e = tid; e < p.experts; e += kThreads) {
    const int lo = __ldg(p.m_indptr + e), hi = __ldg(p.m_indptr + e + 1);
    const int first = lo / kTileRows + e;
    const int tiles = (hi - lo + kTileRows - 1) / kTileRows;
    const int atom_row = blockIdx.x;
    if (atom_row >= first && atom_row < first + tiles) {
      const int local = atom_row - first;
      s_tile[0] = lo + local * kTileRows;
      s_tile[1] = min(kTileRows, hi - lo - local * kTileRows);
      s_tile[2] = 1;
    }
  }
  __syncthreads();
  if (s_tile[2] == 0) return;
  const int row0 = s_tile[0], valid = s_tile[1];
  const int row_bytes = p.features >> 4;
  const int byte0 = blockIdx.y * kSwizzleCols;
  const int bytes_here = min(kSwizzleCols, row_bytes - byte0);  // a multiple of 4
  // coalesced load: 8 threads x 16 bytes per row
  for (int i = tid; i < kTileRows * (kSwizzleCols / 16); i += kThreads) {
    const int r = i / (kSwizzleCols / 16), piece = i % (kSwizzleCols / 16);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid && piece * 16 < bytes_here)
      v = *reinterpret_cast<const uint4*>(p.linear + static_cast<int64_t>(row0 + r) * row_bytes + byte0 + piece * 16);
    *reinterpret_cast<uint4*>(&s_rows[r][piece * 16]) = v;
  }
  __syncthreads();
  const int atom_cols = p.features >> 6;
  const int cols_here = bytes_here >> 2;
  for (int i = tid; i < cols_here * 32; i += kThreads) {
    const int c = i >> 5, rr = i & 31;
    uint4 v;
    v.x = *reinterpret_cast<const uint32_t*>(&s_rows[rr][c * 4]);
    v.y = *reinterpret_cast<const uint32_t*>(&s_rows[rr + 32][c * 4]);
    v.z = *reinterpret_cast<const uint32_t*>(&s_rows[rr + 64][c * 4]);
    v.w = *reinterpret_cast<const uint32_t*>(&s_rows[rr + 96][c * 4]);
    uint8_t* dst = p.atoms + (static_cast<int64_t>(blockIdx.x) * atom_cols + (byte0 >> 2) + c) * 512 + rr * 16;
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

// ------------------------------------------------ cross-rank signal: exchange and barrier
// One CTA per rank.  Optionally stores this rank's per-expert row counts into every rank's
// gathered table, then tells every rank "I am at `epoch`" (one release store into each
// rank's signal pad) and waits until every rank has said the same (acquire loads of its own
// pad).  Everything this rank stored to peer memory in earlier launches of the stream is
// ordered before the signal.  The wait is bounded (ten seconds unless the caller says
// otherwise): when it runs out the kernel sets the status bit LM_STATUS_EP_TIMEOUT and
// returns.  Ranks must run on different GPUs.
constexpr long long kCyclesPerMs = 2000000ll;  // at about 2 GHz

struct SignalParams {
  const int32_t* m_indptr;  // nullptr: barrier only
  int experts;
  int world;
  int rank;
  long long wait_cycles;
  int32_t* counts_all[kMaxRanks];  // every rank's (world, experts) table
  uint32_t* signal[kMaxRanks];     // every rank's pad of `world` words
};

__global__ void __launch_bounds__(256) ep_signal_kernel(SignalParams p) {
  __shared__ uint32_t s_epoch;
  const int tid = threadIdx.x;
  // The epoch is this rank's count of signal calls, kept in word `world` of its own pad, so
  // that a captured CUDA graph can be replayed: every rank makes the same calls in the same
  // order, so the counts agree.
  if (tid == 0) {
    uint32_t* counter = p.signal[p.rank] + p.world;
    s_epoch = *counter + 1;
    *counter = s_epoch;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (p.m_indptr != nullptr) {
    for (int i = tid; i < p.experts; i += blockDim.x) {
      const int count = __ldg(p.m_indptr + i + 1) - __ldg(p.m_indptr + i);
      for (int g = 0; g < p.world; ++g) p.counts_all[g][p.rank * p.experts + i] = count;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.world) {
    uint32_t* theirs = p.signal[tid] + p.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const uint32_t* mine = p.signal[p.rank] + tid;
    const long long start = clock64();
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int32_t>(seen - epoch) >= 0) break;
      if (clock64() - start > p.wait_cycles) {
        atomicOr(&g_ep_status, static_cast<uint32_t>(LM_STATUS_EP_TIMEOUT));
        break;
      }
    }
  }
}

}  // namespace

int ep_status_read(uint32_t* out) {
  LM_CUDA(cudaMemcpyFromSymbol(out, g_ep_status, sizeof(uint32_t)));
  return LM_OK;
}

int ep_status_clear() {
  const uint32_t zero = 0;
  LM_CUDA(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(uint32_t)));
  return LM_OK;
}

}  // namespace lm

extern "C" int lm_ep_plan(const int32_t* counts_all, int world, int rank, int experts, int64_t max_rows,
                          int64_t row_bytes, const uint64_t* return_base, int32_t* own_indptr,
                          int32_t* dest_base, int32_t* owner_start, uint64_t* row_ptrs, int32_t* out_blocks,
                          int32_t* valid, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(counts_all && return_base && own_indptr && dest_base && owner_start && row_ptrs && valid,
             "ep_plan: null pointer");
  LM_REQUIRE(world >= 1 && world <= kMaxRanks, "ep_plan: 1..8 ranks");
  LM_REQUIRE(rank >= 0 && rank < world, "ep_plan: rank out of range");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts && experts % world == 0,
             "ep_plan: 1..256 experts, divisible by the number of ranks");
  LM_REQUIRE(max_rows > 0 && max_rows < (1ll << 31) && row_bytes > 0 && row_bytes % 16 == 0,
             "ep_plan: bad buffer geometry");
  PlanParams p{};
  p.counts_all = counts_all;
  p.world = world;
  p.rank = rank;
  p.experts = experts;
  p.local_experts = experts / world;
  p.max_rows = max_rows;
  p.row_bytes = row_bytes;
  for (int g = 0; g < world; ++g) p.return_base[g] = return_base[g];
  p.own_indptr = own_indptr;
  p.dest_base = dest_base;
  p.owner_start = owner_start;
  p.row_ptrs = row_ptrs;
  p.out_blocks = out_blocks;
  p.valid = valid;
  const int segments = p.local_experts * world;
  ep_plan_kernel<<<segments < 296 ? segments : 296, kPlanThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_ep_quantize_send(const void* x, int64_t tokens, int features, int top_k, int world,
                                   int experts, const int32_t* slots, const int32_t* topk_ids,
                                   const int32_t* src_indptr, const int32_t* dest_base,
                                   const int32_t* owner_start, const int32_t* valid,
                                   const float* scale_pair, const uint64_t* q_base,
                                   const uint64_t* sf_base, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(x && slots && topk_ids && src_indptr && dest_base && owner_start && valid && scale_pair &&
                 q_base && sf_base,
             "ep_quantize_send: null pointer");
  LM_REQUIRE(features > 0 && features % 64 == 0, "ep_quantize_send: features must be a multiple of 64");
  LM_REQUIRE(top_k > 0 && top_k <= 32 && tokens >= 0, "ep_quantize_send: bad sizes");
  LM_REQUIRE(world >= 1 && world <= kMaxRanks && experts > 0 && experts % world == 0,
             "ep_quantize_send: bad rank or expert count");
  if (tokens == 0) return LM_OK;
  SendParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.tokens = tokens;
  p.features = features;
  p.top_k = top_k;
  p.local_experts = experts / world;
  p.slots = slots;
  p.topk_ids = topk_ids;
  p.src_indptr = src_indptr;
  p.dest_base = dest_base;
  p.owner_start = owner_start;
  p.valid = valid;
  p.scale_pair = scale_pair;
  for (int g = 0; g < world; ++g) {
    LM_REQUIRE(q_base[g] != 0 && sf_base[g] != 0 && q_base[g] % 16 == 0 && sf_base[g] % 16 == 0,
               "ep_quantize_send: peer buffers must be 16-byte aligned");
    p.q[g] = reinterpret_cast<uint8_t*>(q_base[g]);
    p.sf[g] = reinterpret_cast<uint8_t*>(sf_base[g]);
  }
  dim3 grid(static_cast<unsigned>((tokens + kWarps - 1) / kWarps));
  ep_quantize_send_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_ep_sf_swizzle(const uint8_t* linear, int64_t max_rows, int features,
                                const int32_t* m_indptr, int experts, uint8_t* atoms,
                                lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(linear && m_indptr && atoms, "ep_sf_swizzle: null pointer");
  LM_REQUIRE(features > 0 && features % 64 == 0, "ep_sf_swizzle: features must be a multiple of 64");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts && max_rows > 0, "ep_sf_swizzle: bad sizes");
  LM_REQUIRE((reinterpret_cast<uintptr_t>(linear) & 15) == 0 && (reinterpret_cast<uintptr_t>(atoms) & 15) == 0 &&
                 (features / 16) % 16 == 0,
             "ep_sf_swizzle: buffers and rows must be 16-byte aligned (features a multiple of 256)");
  SwizzleParams p{linear, m_indptr, experts, features, atoms};
  const int64_t atom_rows = (max_rows + kTileRows - 1) / kTileRows + experts;
  dim3 grid(static_cast<unsigned>(atom_rows), (features / 16 + kSwizzleCols - 1) / kSwizzleCols);
  ep_sf_swizzle_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_ep_signal(const int32_t* m_indptr, int experts, int world, int rank,
                            const uint64_t* counts_all_base, const uint64_t* signal_base, int timeout_ms,
                            lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(signal_base, "ep_signal: null pointer");
  LM_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "ep_signal: bad rank");
  LM_REQUIRE(m_indptr == nullptr || (counts_all_base != nullptr && experts > 0 && experts <= kMaxExperts),
             "ep_signal: the count exchange needs the gathered tables");
  SignalParams p{};
  p.m_indptr = m_indptr;
  p.experts = experts;
  p.world = world;
  p.rank = rank;
  LM_REQUIRE(timeout_ms >= 0 && timeout_ms <= 60000, "ep_signal: timeout of 0 (default) to 60000 ms");
  p.wait_cycles = (timeout_ms > 0 ? timeout_ms : 10000) * kCyclesPerMs;
  for (int g = 0; g < world; ++g) {
    LM_REQUIRE(signal_base[g] != 0 && signal_base[g] % 4 == 0, "ep_signal: bad signal pad");
    p.signal[g] = reinterpret_cast<uint32_t*>(signal_base[g]);
    if (m_indptr != nullptr) {
      LM_REQUIRE(counts_all_base[g] != 0 && counts_all_base[g] % 4 == 0, "ep_signal: bad count table");
      p.counts_all[g] = reinterpret_cast<int32_t*>(counts_all_base[g]);
    }
  }
  ep_signal_kernel<<<1, 256, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
