// Persistent grouped / dense NVFP4 GEMM for sm_100a.
//
//   out[rows_e, :] = alpha_e * (A_e . SFA_e) (B_e . SFB_e)^T      FP32 accumulate
//
// Warp-specialised CTA of 384 threads, one CTA per SM:
//   warp 0       TMA producer: A and B tiles (128-byte swizzle) with
//                cp.async.bulk.tensor, scale-factor atoms with cp.async.bulk
//   warp 1       allocates TMEM; one elected thread issues, per 64-element chunk, the
//                tcgen05.cp copies that bring the chunk's scale-factor atoms from shared
//                memory to TMEM and then the tcgen05.mma kind::mxf4nvf4 block-scaled MMA
//                (copies and MMAs of one thread run in issue order)
//   warp 2       tile prefix table at start-up
//   warps 4..11  epilogue in two groups of four: tcgen05.ld a 64-column slice of the
//                accumulator, scale, (activate and requantize to NVFP4,) store; each warp
//                owns one TMEM lane quarter.  BF16 blocks of 32 whole rows leave through a
//                TMA store from swizzled staging
// Tiles are 128 x 128 (two accumulators in TMEM, group g drains accumulator g) or 128 x 256
// (two accumulators that overlap in TMEM, both groups on every tile): see gemm_kernel.
// gemm_pair_kernel runs 256 x 256 tiles on pairs of CTAs with tcgen05.mma.cta_group::2.
//
// Work is cut into units of one row tile times a run of column tiles and dealt round-robin
// to the CTAs.  With 128-column tiles and a short contraction (K <= 2048) the A tile and its
// scale factors stay resident in shared memory for the whole unit and only B streams
// through the ring; otherwise A and B stream together and a unit is a single tile.  Every
// role derives the same unit list from m_indptr in shared memory.
//
// Rows of expert e are [m_indptr[e], m_indptr[e+1]).  A tile's A rows may run
// into the next expert (or past the end, where TMA fills zeros); those rows are
// computed and then not stored.  Every wait on an mbarrier is bounded: when it
// runs out the CTA raises a bit in a status word and leaves the kernel.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace lm {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kStageKBytes = 128;  // 256 FP4 values per row and stage: one swizzle span
constexpr int kChunksPerStage = 4; // 64-element MMAs (= scale-factor atoms) per stage
constexpr int kEpilogueWarps = 8;
constexpr int kFirstEpilogueWarp = 4;  // warps 4..11: two epilogue groups of four (warp & 3 = TMEM lane quarter)
constexpr int kThreads = 32 * (kFirstEpilogueWarp + kEpilogueWarps);
constexpr int kMaxExperts = 256;
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitLimitCycles = 2000000000ll;  // about one second
constexpr int kMaxDevices = 64;  // per-device caches of host-side state

// shared memory: operand slots of 18 KB (a 128 x 128 B tile + its 2 KB of scale factors)
constexpr int kTileBytes = kTileM * kStageKBytes;        // 16384
constexpr int kSfBytes = kChunksPerStage * 512;          // 2048
constexpr int kSlotBytes = kTileBytes + kSfBytes;        // 18432
constexpr int kMaxRing = 8;      // ring stages (128-column tiles: also TMEM scale-factor slots)
constexpr int kMaxResident = 8;  // resident A stages: K <= 2048
constexpr int kStoreRowPitch = 64 * 2;                   // BF16 staging row: 64 columns, 128-byte swizzled
constexpr int kStoreBytesPerWarp = 32 * kStoreRowPitch;  // 4 KB: four swizzle atoms of 8 rows
constexpr int kStoreBytes = kEpilogueWarps * kStoreBytesPerWarp;
constexpr int kMiscBytes = 4096;
constexpr int kSmemLimit = 232448;
constexpr uint32_t kSfCol = 2 * kTileN;  // TMEM: two accumulators, then 32 columns per ring stage
// TMEM with 256-column tiles: two 256-column accumulators and the scale factors do not fit in
// 512 columns side by side, so the accumulators overlap: accumulator 0 at [0, 256), accumulator
// 1 at [192, 448), the scale factors of one stage in 48 columns from 448.  The overlap is
// exactly one 64-column slice (slice 3 of accumulator 0, slice 0 of accumulator 1): it alone
// stands between the end of a tile's MMAs and the start of the next tile's, and four epilogue
// warps own it.  (An accumulator that does not start on a multiple of 32 columns made every
// TMEM load slower.)
constexpr uint32_t kWideAcc1Col = 192;
constexpr uint32_t kWideSfCol = 448;
constexpr uint32_t kWideSharedOwners = 4;  // epilogue warps of one CTA that arrive on `shared_cols_free`
static_assert(kSlotBytes % 1024 == 0, "operand slots must keep 1024-byte alignment");
static_assert(kSfCol + kMaxRing * 32 <= kTmemCols, "TMEM budget");

__host__ __device__ constexpr int data_slots(int out_kind) {
  return (kSmemLimit - 1024 - kMiscBytes - (out_kind == LM_OUT_BF16 ? kStoreBytes : 0)) / kSlotBytes;
}
__host__ __device__ constexpr int smem_bytes(int out_kind) {
  return 1024 + kMiscBytes + (out_kind == LM_OUT_BF16 ? kStoreBytes : 0) + data_slots(out_kind) * kSlotBytes;
}

__device__ uint32_t g_status = 0;


enum : uint32_t {
  kStatusProducerTimeout = 1u,
  kStatusMmaTimeout = 2u,
  kStatusEpilogueTimeout = 4u,  // (8 was the scale-factor warps' bit; 16 belongs to the cross-rank signal)
};

struct GemmParams {
  int experts;
  int n;
  int n_tiles;
  int k_stages;
  int atom_cols;      // k / 64
  int sfb_atom_rows;  // ceil(n / 128)
  int dense;
  int alpha_per_expert;
  int a_resident;     // 1: A stays in shared memory for a whole unit
  int ring_stages;    // stages of the streaming ring
  int n_per_unit;     // column tiles per unit
  int units_per_mtile;
  int64_t rows;
  const int32_t* m_indptr;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  void* out;
  uint8_t* out_sf;
  const float* out_scale;
  const uint64_t* out_row_ptrs;  // BF16 output: optional address of every output row
  const int32_t* out_blocks;     // with out_row_ptrs: (tile atom row * 4 + quarter) -> {rank, first row} or -1
  int tma_store;                 // BF16 output: whole 32-row blocks leave through TMA stores
  int uneven;                    // BF16 / FP32 output, 256-column tiles: uneven split of the epilogue
  int out_atom_cols;  // NVFP4 output: out_n / 64
  float clamp_limit;
  float sigmoid_alpha;
  float up_bias;
};

// ------------------------------------------------------------------ PTX glue
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false when the CTA is aborting (this wait ran out, or
// another role's did); the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t who) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicOr(&g_status, who);
      return false;
    }
  }
}

// Abort path only: wait for a phase without touching the abort flag, for at most `limit` cycles.
__device__ __forceinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity, long long limit) {
  const long long start = clock64();
  while (!mbar_try(bar, parity))
    if (clock64() - start > limit) return false;
  return true;
}

// True in exactly one lane of a converged warp.  Issuing TMA and tcgen05 instructions under
// this predicate (instead of `lane == 0`) lets the compiler keep their operands in uniform
// registers: the surrounding control flow stays warp-uniform.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// 32 rows x 64 BF16 columns from swizzled shared memory to global memory; out-of-range columns
// and rows are clipped by the tensor map.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The stores issued so far have read their shared memory / have completed.
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tc_wait_ld_regs(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of
// 128 bytes, eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// Instruction descriptor: E2M1 x E2M1, UE4M3 scale factors, K-major A and B,
// M = 128, N = n, K = 64, FP32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (0u << 23) |
         (static_cast<uint32_t>(kTileM >> 4) << 24);
}

// Tensor maps of the return buffers of the ranks of an expert-parallel group (BF16 rows that go
// back to the rank that sent them): 32-row x 64-column boxes like the local output map.
struct ReturnMaps {
  CUtensorMap rank[LM_EP_MAX_RANKS];
};

struct Misc {  // lives after the operand slots and the store staging
  uint64_t full[kMaxRing];         // ring stage filled by TMA
  uint64_t empty[kMaxRing];        // ring stage drained by the MMAs
  uint64_t a_full[kMaxResident];   // resident A stage filled
  uint64_t a_empty[kMaxResident];  // resident A stage no longer read
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t shared_cols_free;       // 256-column tiles: the columns both accumulators use are read out
  uint64_t drain;                  // abort path: the MMAs issued so far have completed
  uint32_t tmem_base;
  int abort_flag;
  int total_m_tiles;
  int fills_issued;                // abort path: ring / resident-A fills the producer started ...
  int fills_taken;                 // ... and those the MMA warp saw complete
  int a_fills_issued;
  int a_fills_taken;
  int pad;
  int cu[kMaxExperts + 1];
  int prefix[kMaxExperts + 2];
};
static_assert(sizeof(Misc) <= kMiscBytes, "misc block too large");

struct RowTile {
  int expert;
  int row0;    // first A / out row of the tile
  int valid;   // rows of the tile that belong to the expert
  int sf_row;  // scale-factor atom row of the tile
};

// Maps a row-tile index to its expert.  A role visits row tiles in increasing order, so
// the expert cursor only moves forward.
struct TileWalker {
  int expert = 0;
  __device__ __forceinline__ RowTile at(const Misc* m, const GemmParams& p, int mt) {
    while (expert + 1 < p.experts && m->prefix[expert + 1] <= mt) ++expert;
    const int local = mt - m->prefix[expert];
    const int begin = m->cu[expert];
    const int count = m->cu[expert + 1] - begin;
    RowTile t;
    t.expert = expert;
    t.row0 = begin + local * kTileM;
    t.valid = min(kTileM, count - local * kTileM);
    t.sf_row = begin / kTileM + expert + local;
    return t;
  }
};

// The column-tile run [n_begin, n_end) of row tile mt that makes up one unit.
struct Unit {
  int mt;
  int n_begin;
  int n_end;
};
__device__ __forceinline__ Unit decode_unit(const GemmParams& p, int unit) {
  Unit u;
  u.mt = unit / p.units_per_mtile;
  u.n_begin = (unit - u.mt * p.units_per_mtile) * p.n_per_unit;
  u.n_end = min(u.n_begin + p.n_per_unit, p.n_tiles);
  return u;
}

// ------------------------------------------------------------- activations
template <int kAct>
__device__ __forceinline__ float gated_value(float g, float u, float clamp_limit, float sigmoid_alpha,
                                             float up_bias) {
  if (clamp_limit > 0.0f) {
    g = fminf(g, clamp_limit);
    u = fmaxf(fminf(u, clamp_limit), -clamp_limit);
  }
  if (kAct == LM_ACT_SWIGLU || kAct == LM_ACT_SWIGLU_OAI) {
    // exp(-a g) as fast-math exp computes it, 2^(x log2 e) with both roundings.  The flushing
    // form of ex2 only differs where the result is a denormal, which the add of 1 absorbs, and
    // it spares the scaling instructions around the plain form; plain swiglu has a = 1.
    const float x = kAct == LM_ACT_SWIGLU ? -g : -sigmoid_alpha * g;
    float e, sig;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sig) : "f"(1.0f + e));
    return g * sig * (u + up_bias);
  }
  if (kAct == LM_ACT_GEGLU) {
    const float root = 0.7978845608028654f;  // sqrt(2/pi)
    float arg = root * (g + 0.044715f * g * g * g);
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(arg));
    return 0.5f * g * (1.0f + th) * u;
  }
  return fmaxf(g, 0.0f) * u;  // reglu
}

// Two FP32 products in one instruction (round to nearest, as two separate multiplies give).
__device__ __forceinline__ void mul_pair(float& a, float& b, float s) {
  asm("{\n\t.reg .b64 v, f;\n\tmov.b64 v, {%0, %1};\n\tmov.b64 f, {%2, %2};\n\t"
      "mul.rn.f32x2 v, v, f;\n\tmov.b64 {%0, %1}, v;\n\t}"
      : "+f"(a), "+f"(b)
      : "f"(s));
}

// Requantize 16 post-activation values: returns the E4M3 byte, packs 8 bytes.
__device__ __forceinline__ uint32_t requant16(const float* h, float inv_pts, uint32_t* packed) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(h[i]));
  const float scaled = amax * (inv_pts * inv6());
  const uint32_t sf = f32_to_e4m3(scaled);
  float rescale;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rescale) : "f"(e4m3_to_f32(sf)));
  rescale = fminf(rescale * inv_pts, kFltMax);
  float s[16];
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    s[i] = h[i];
    s[i + 1] = h[i + 1];
    mul_pair(s[i], s[i + 1], rescale);
  }
  packed[0] = f32x8_to_e2m1(s);
  packed[1] = f32x8_to_e2m1(s + 8);
  return sf;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&b);
}

// ------------------------------------------------------------ epilogue of one tile
// What an epilogue warp needs to drain its share of one accumulator.
struct DrainContext {
  uint32_t lane_base;        // TMEM address of the warp's 32 lanes, column 0
  uint32_t warp_store;       // the warp's BF16 staging in shared memory (1024-byte aligned)
  const CUtensorMap* out_map;  // BF16 output: tensor map of the output (32 x 64 boxes)
  const ReturnMaps* return_maps;  // BF16 output through out_blocks: the ranks' return buffers
  uint32_t bar_shared_cols;  // signalled when the columns both accumulators use are in registers
  uint32_t bar_acc_empty;    // signalled when the whole accumulator is in registers
  bool remote;               // the two barriers are cluster addresses (the pair leader's)
  uint32_t acc1_col;         // 256-column tiles: first TMEM column of accumulator 1
  int group;                 // epilogue group of the warp (0 or 1)
  int quarter;               // TMEM lane quarter of the warp
  int lane;
  float alpha;
  float inv_h;               // NVFP4 output: reciprocal of the output's tensor scale
};

// Arrive on a barrier of this CTA or, `remote`, of the pair's leader (a cluster address).  The
// remote form is relaxed: every use orders accesses to TMEM, which tcgen05.wait::ld/st and the
// tcgen05 fences on both sides cover, and an arrive with cluster-scope release semantics took
// thousands of cycles here (the MMAs then spent most of their time waiting for it).
__device__ __forceinline__ void signal_barrier(uint32_t bar, bool remote) {
  if (remote) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
  } else {
    mbar_arrive(bar);
  }
}

template <int kOut, int kAct, int kNB>
__device__ __forceinline__ void drain_tile(const GemmParams& p, const RowTile& t, const DrainContext& c,
                                           const int acc, const int nt) {
  const uint32_t lane_base = c.lane_base;
  const uint32_t warp_store = c.warp_store;
  (void)warp_store;
  const int group = c.group, quarter = c.quarter, lane = c.lane;
  const float alpha = c.alpha, inv_h = c.inv_h;
  (void)inv_h;
  const bool row_ok = quarter * 32 + lane < t.valid;
  const int64_t out_row = static_cast<int64_t>(t.row0) + quarter * 32 + lane;
  const uint32_t taddr = lane_base + acc * (kNB == 1 ? kTileN : c.acc1_col);

  // The 64-column slices this warp drains, first to last, four bits each.  With 256-column
  // tiles the MMAs of the next tile wait until the slice that holds the columns the other
  // accumulator also uses (slice 3 of accumulator 0, slice 0 of accumulator 1) is in registers,
  // and a warp that is still busy with the previous tile cannot release the next one.
  //  * uneven split: group 1 drains nothing but the shared slice, so it is idle again long
  //    before the next tile ends, and group 0 the other three.  NVFP4 output always: the gated
  //    activation and the requantization keep both warps of a scheduler on its
  //    special-function unit, whose work per tile is the same however the slices are dealt.
  //    BF16 / FP32 output when the K loop is long enough to cover a three-slice drain
  //    (`p.uneven`, set by the host): 3 to 8 % faster at K = 2048, 9 % slower at K = 512.
  //  * even split: two slices each; the group whose first slice is the shared one owns it.
  const bool uneven = kNB == 2 && (kOut == LM_OUT_NVFP4 || p.uneven != 0);
  uint32_t slices;
  int count = 2;
  bool owns_shared = false;
  if (kNB == 1) {
    slices = 0x10u;
  } else if (uneven) {
    if (group == 1) {
      slices = acc == 0 ? 0x3u : 0x0u;
      count = 1;
      owns_shared = true;
    } else {
      slices = acc == 0 ? 0x210u : 0x321u;
      count = 3;
    }
  } else if (acc == 0) {
    slices = group == 1 ? 0x13u : 0x02u;
    owns_shared = group == 1;
  } else {
    slices = group == 1 ? 0x31u : 0x20u;
    owns_shared = group == 0;
  }
  const int first = static_cast<int>(slices & 0xFu);
  auto slice_at = [&](int s) { return static_cast<int>((slices >> (4 * s)) & 0xFu); };
  const bool rows_any = t.valid > quarter * 32;  // this warp owns at least one valid row
  // rows may live anywhere (another GPU's buffer): lane l holds the address of row l
  unsigned long long row_base = 0;
  // where this warp's 32-row block goes when it leaves as one bulk store: the output itself, or
  // the return buffer of the rank the route plan names for it
  const CUtensorMap* block_map = nullptr;
  int block_row = 0;
  if (kOut == LM_OUT_BF16) {
    if (p.out_row_ptrs == nullptr) {
      if (p.tma_store && t.valid - quarter * 32 >= 32) {
        block_map = c.out_map;
        block_row = t.row0 + quarter * 32;
      }
    } else {
      if (p.out_blocks != nullptr && t.valid - quarter * 32 >= 32) {
        const int2 dst = __ldg(reinterpret_cast<const int2*>(p.out_blocks) + (t.sf_row * 4 + quarter));
        if (dst.x >= 0) {
          block_map = &c.return_maps->rank[dst.x];
          block_row = dst.y;
        }
      }
      if (block_map == nullptr && quarter * 32 + lane < t.valid)
        row_base = __ldg(reinterpret_cast<const unsigned long long*>(p.out_row_ptrs) + t.row0 + quarter * 32 + lane);
    }
  }
  uint32_t va[32], vb[32];
  int cur = first;
  tc_load32(taddr + cur * 64, va);
  tc_load32(taddr + cur * 64 + 32, vb);
  tc_wait_ld_regs(va);
  tc_wait_ld_regs(vb);
  // the first slice is in registers: if it is the shared one, the next tile's MMAs may start;
  // if it is the only one, the warp is done reading the accumulator
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    if (kNB == 2 && owns_shared) signal_barrier(c.bar_shared_cols, c.remote);
    if (count == 1) signal_barrier(c.bar_acc_empty, c.remote);
  }

  // ---- per-slice state and the two halves of the work
  constexpr bool kGated = kAct != LM_ACT_RELU2;
  uint32_t q[8];   // NVFP4: packed codes of the slice
  uint32_t sfw = 0;  // NVFP4: scale-factor bytes of the slice
  (void)q;
  (void)sfw;
  auto convert = [&](const uint32_t* v, const int half, const int col64) {
    if (kOut == LM_OUT_NVFP4) {
      if (kGated) {
        // 32 accumulator columns = 16 (gate, up) pairs -> 16 outputs: 8 bytes, one factor
        float h[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float g = __uint_as_float(v[2 * i]), u = __uint_as_float(v[2 * i + 1]);
          mul_pair(g, u, alpha);
          h[i] = gated_value<kAct>(g, u, p.clamp_limit, p.sigmoid_alpha, p.up_bias);
        }
        const uint32_t sf = requant16(h, inv_h, &q[2 * half]);
        sfw = half == 0 ? sf : (sfw | (sf << 8));
      } else {
        // 32 outputs: 16 bytes, two factors
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float h[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x = fmaxf(__uint_as_float(v[16 * c + i]) * alpha, 0.0f);
            h[i] = x * x;
          }
          const uint32_t sf = requant16(h, inv_h, &q[4 * half + 2 * c]);
          sfw = (half == 0 && c == 0) ? sf : (sfw | (sf << (8 * (2 * half + c))));
        }
      }
    } else if (kOut == LM_OUT_BF16) {
      // lane = row: the warp's 32 x 64 block goes to its shared-memory staging, 16-byte chunk c
      // of row r at chunk c ^ (r % 8) (the 128-byte swizzle the output tensor map expects; it
      // also keeps these stores and the transposed loads free of bank conflicts)
      if (half == 0) {
        // the previous slice's TMA store must have read the staging
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(warp_store + lane * kStoreRowPitch +
                                                                       (((half * 4 + i) ^ (lane & 7)) * 16)),
                     "r"(pack_bf16x2(__uint_as_float(v[8 * i]) * alpha, __uint_as_float(v[8 * i + 1]) * alpha)),
                     "r"(pack_bf16x2(__uint_as_float(v[8 * i + 2]) * alpha, __uint_as_float(v[8 * i + 3]) * alpha)),
                     "r"(pack_bf16x2(__uint_as_float(v[8 * i + 4]) * alpha, __uint_as_float(v[8 * i + 5]) * alpha)),
                     "r"(pack_bf16x2(__uint_as_float(v[8 * i + 6]) * alpha, __uint_as_float(v[8 * i + 7]) * alpha))
                     : "memory");
    } else {
      float* out_base = static_cast<float*>(p.out) + out_row * p.n + col64 * 64 + half * 32;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // N is a multiple of 8: groups of four never straddle the edge
        if (row_ok && col64 * 64 + half * 32 + 4 * i < p.n)
          reinterpret_cast<float4*>(out_base)[i] =
              make_float4(__uint_as_float(v[4 * i]) * alpha, __uint_as_float(v[4 * i + 1]) * alpha,
                          __uint_as_float(v[4 * i + 2]) * alpha, __uint_as_float(v[4 * i + 3]) * alpha);
      }
    }
  };
  auto finish = [&](const int col64) {
    const bool cols_ok = col64 * 64 < p.n;
    if (kOut == LM_OUT_NVFP4) {
      const int out_n = p.out_atom_cols * 64;
      if (row_ok && cols_ok) {
        if (kGated) {
          uint8_t* codes = static_cast<uint8_t*>(p.out) + out_row * (out_n >> 1) +
                           static_cast<int64_t>(col64) * 16;
          *reinterpret_cast<uint4*>(codes) = make_uint4(q[0], q[1], q[2], q[3]);
          uint8_t* dst = p.out_sf +
                         (static_cast<int64_t>(t.sf_row) * p.out_atom_cols + (col64 >> 1)) * 512 +
                         lane * 16 + quarter * 4 + (col64 & 1) * 2;
          *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(sfw);
        } else {
          uint8_t* codes = static_cast<uint8_t*>(p.out) + out_row * (out_n >> 1) +
                           static_cast<int64_t>(col64) * 32;
          reinterpret_cast<uint4*>(codes)[0] = make_uint4(q[0], q[1], q[2], q[3]);
          reinterpret_cast<uint4*>(codes)[1] = make_uint4(q[4], q[5], q[6], q[7]);
          uint8_t* dst = p.out_sf +
                         (static_cast<int64_t>(t.sf_row) * p.out_atom_cols + col64) * 512 +
                         lane * 16 + quarter * 4;
          *reinterpret_cast<uint32_t*>(dst) = sfw;
        }
      }
    } else if (kOut == LM_OUT_BF16) {
      const int rows_here = t.valid - quarter * 32;  // valid rows among this warp's 32
      if (block_map != nullptr) {
        // the whole block has one destination: one TMA store moves it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && cols_ok) tma_store_2d(block_map, warp_store, col64 * 64, block_row);
        return;
      }
      // transposed read: a global store covers four whole 128-byte row pieces
      __syncwarp();
      if (rows_any && cols_ok) {
        __nv_bfloat16* warp_out =
            static_cast<__nv_bfloat16*>(p.out) + (static_cast<int64_t>(t.row0) + quarter * 32) * p.n;
        const int piece = lane & 7;
        const int col = col64 * 64 + piece * 8;
        uint4 d[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(d[i].x), "=r"(d[i].y), "=r"(d[i].z), "=r"(d[i].w)
                       : "r"(warp_store + (4 * i + (lane >> 3)) * kStoreRowPitch +
                             ((piece ^ ((4 * i + (lane >> 3)) & 7)) * 16)));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = 4 * i + (lane >> 3);
          __nv_bfloat16* dst = warp_out + static_cast<int64_t>(row) * p.n;
          if (p.out_row_ptrs != nullptr)
            dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xFFFFFFFFu, row_base, row));
          if (row < rows_here && col < p.n) *reinterpret_cast<uint4*>(dst + col) = d[i];
        }
      }
      __syncwarp();
    }
  };

  // Software pipeline over the 32-column halves of the slices: while a half is converted, the
  // load of the half after next is in flight (a TMEM load takes several hundred cycles from
  // issue to data).
  auto step = [&](const bool more, const bool last_load, const int next) {
    const int col = nt * 2 * kNB + cur;
    convert(va, 0, col);
    if (more) tc_load32(taddr + next * 64, va);
    convert(vb, 1, col);
    if (more) tc_load32(taddr + next * 64 + 32, vb);
    finish(col);
    if (more) {
      tc_wait_ld_regs(va);
      tc_wait_ld_regs(vb);
      if (last_load) {
        // the warp's last slice is in registers: it has read all it reads of the accumulator
        tc_fence_before();
        __syncwarp();
        if (lane == 0) signal_barrier(c.bar_acc_empty, c.remote);
      }
      cur = next;
    }
  };
  if (count == 2) {
    // straight-line code for the common case
    step(true, true, slice_at(1));
    step(false, false, 0);
  } else {
#pragma unroll 1
    for (int s = 0; s < count; ++s) step(s + 1 < count, s + 2 == count, s + 1 < count ? slice_at(s + 1) : 0);
  }
}

// Shared-memory descriptor of one 512-byte scale-factor atom: 32 rows of 16 bytes, no swizzle,
// eight-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf_atom(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(128 >> 4) << 32;               // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  return d;
}

// One scale-factor atom from shared memory into four TMEM columns, the 32 rows repeated in all
// four lane quarters (the layout the block-scaled MMA reads).  Runs in issue order with the
// MMAs of the same thread.
__device__ __forceinline__ void tc_copy_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Programmatic dependent launch of the prefill kernels (short steps: a handful of launches of a
// few microseconds each, where a kernel's set-up can run beside its predecessor).  The wait comes
// after barriers and TMEM are set up and before anything an earlier kernel wrote is read; the
// kernel's own dependents are released only after it, so a kernel past its wait knows that
// every older kernel is complete.  Launched the plain way both instructions do nothing.
__device__ __forceinline__ void prefill_pdl_wait_and_release() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------ kernel
// kNB = 128-column blocks per tile.
// 1: 128 x 128 tiles, two accumulators of 128 TMEM columns, one scale-factor slot per ring
//    stage; epilogue group g drains accumulator g (every other tile).
// 2: 128 x 256 tiles, which move a quarter less data through shared memory per FLOP (the
//    resource that binds the main loop).  Two 256-column accumulators and the scale factors
//    do not fit in 512 TMEM columns side by side, so the accumulators overlap in 48 columns:
//    both epilogue groups work on every tile, the owner of the 64-column slice that touches
//    the overlap reads it first and signals `shared_cols_free`; the MMAs of the next tile
//    start then, while the rest of the tile is still being converted and stored.
template <int kOut, int kAct, int kNB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a64,
            const __grid_constant__ CUtensorMap tmap_a32, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ ReturnMaps tmap_return,
            const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kSlots = data_slots(kOut);
  const uint32_t store_base = smem_base + kSlots * kSlotBytes;
  Misc* misc = reinterpret_cast<Misc*>(smem_gen + kSlots * kSlotBytes +
                                       (kOut == LM_OUT_BF16 ? kStoreBytes : 0));
  volatile int* abort_flag = &misc->abort_flag;

  // operand slots: [resident A stages][ring stages]; a ring stage is B (+ A when streaming)
  const bool resident = kNB == 1 && p.a_resident != 0;
  // ring stage: [B tile(s)][B scale factors][A tile][A scale factors]
  const uint32_t ring_base = smem_base + (resident ? p.k_stages * kSlotBytes : 0);
  const uint32_t ring_stride = (resident ? kNB : kNB + 1) * kSlotBytes;
  constexpr uint32_t kSfbOffset = kNB * kTileBytes;   // within a ring stage
  constexpr uint32_t kAOffset = kNB * kSlotBytes;     // streaming only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- one-time setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxRing; ++s) {
      mbar_init(smem_u32(&misc->full[s]), 1);
      mbar_init(smem_u32(&misc->empty[s]), 1);
    }
    for (int s = 0; s < kMaxResident; ++s) {
      mbar_init(smem_u32(&misc->a_full[s]), 1);
      mbar_init(smem_u32(&misc->a_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&misc->acc_full[s]), 1);
      mbar_init(smem_u32(&misc->acc_empty[s]), kNB == 1 ? 4 : 8);
    }
    mbar_init(smem_u32(&misc->shared_cols_free), kWideSharedOwners);
    mbar_init(smem_u32(&misc->drain), 1);
    misc->abort_flag = 0;
    misc->fills_issued = misc->fills_taken = misc->a_fills_issued = misc->a_fills_taken = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&misc->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  prefill_pdl_wait_and_release();
  // expert boundaries -> shared memory (volatile loads: one the compiler knows as invariant
  // could move above the wait)
  if (p.dense) {
    if (threadIdx.x == 0) {
      misc->cu[0] = 0;
      misc->cu[1] = static_cast<int>(p.rows);
    }
  } else {
    for (int e = threadIdx.x; e <= p.experts; e += kThreads)
      misc->cu[e] = *reinterpret_cast<const volatile int32_t*>(p.m_indptr + e);
  }
  __syncthreads();
  if (warp == 2) {
    // exclusive prefix of row tiles per expert; each lane owns 8 experts
    int local[8];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int e = lane * 8 + i;
      int tiles = 0;
      if (e < p.experts) tiles = (misc->cu[e + 1] - misc->cu[e] + kTileM - 1) / kTileM;
      local[i] = sum;
      sum += tiles;
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += t;
    }
    const int base = incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int e = lane * 8 + i;
      if (e < p.experts) misc->prefix[e] = base + local[i];
    }
    if (lane == 31) {
      misc->total_m_tiles = incl;
      misc->prefix[p.experts] = incl;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = misc->tmem_base;
  const int total_units = misc->total_m_tiles * p.units_per_mtile;

  if (warp == 0) {
    // ===================================================== TMA producer
    TileWalker walker;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t a_phase = 0;
    bool ok = true;
    int fills = 0, a_fills = 0;  // loads started: the abort path waits for those nobody consumed
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const Unit u = decode_unit(p, unit);
      const RowTile t = walker.at(misc, p, u.mt);
      const uint8_t* sfa_src = p.sfa + static_cast<int64_t>(t.sf_row) * p.atom_cols * 512;
      // A row tile with few valid rows (decode, expert tails) is fetched with a shorter TMA
      // box; the rest of the 128-row operand keeps stale bytes whose products are never stored
      const CUtensorMap* a_map = t.valid <= 32 ? &tmap_a32 : (t.valid <= 64 ? &tmap_a64 : &tmap_a);
      const uint32_t a_bytes = (t.valid <= 32 ? 32 : (t.valid <= 64 ? 64 : 128)) * kStageKBytes;
      for (int nt = u.n_begin; nt < u.n_end && ok; ++nt) {
        const int b_row = t.expert * p.n + nt * kNB * kTileN;
        const uint8_t* sfb_src =
            p.sfb + static_cast<int64_t>(t.expert * p.sfb_atom_rows + nt * kNB) * p.atom_cols * 512;
        // column blocks of this tile that exist (N need not be a multiple of the tile width)
        const int b_blocks = min(kNB, p.sfb_atom_rows - nt * kNB);
        for (int ks = 0; ks < p.k_stages; ++ks) {
          const int chunks = min(kChunksPerStage, p.atom_cols - ks * kChunksPerStage);
          const uint32_t sf_bytes = chunks * 512;
          if (resident && nt == u.n_begin) {
            // the unit's A tile, stage by stage, as soon as the previous unit has let go of it
            ok = mbar_wait(smem_u32(&misc->a_empty[ks]), a_phase ^ 1u, abort_flag, kStatusProducerTimeout);
            if (!ok) break;
            if (elect_one()) {
              const uint32_t bar = smem_u32(&misc->a_full[ks]);
              const uint32_t dst = smem_base + ks * kSlotBytes;
              mbar_expect_tx(bar, a_bytes + sf_bytes);
              tma_load_2d(dst, a_map, ks * kStageKBytes, t.row0, bar);
              bulk_load(dst + kTileBytes, sfa_src + static_cast<int64_t>(ks) * kSfBytes, sf_bytes, bar);
            }
            __syncwarp();
            ++a_fills;
          }
          ok = mbar_wait(smem_u32(&misc->empty[stage]), phase ^ 1u, abort_flag, kStatusProducerTimeout);
          if (!ok) break;
          if (elect_one()) {
            const uint32_t bar = smem_u32(&misc->full[stage]);
            const uint32_t dst = ring_base + stage * ring_stride;
            mbar_expect_tx(bar, kNB * kTileBytes + b_blocks * sf_bytes + (resident ? 0u : a_bytes + sf_bytes));
            tma_load_2d(dst, &tmap_b, ks * kStageKBytes, b_row, bar);
            for (int j = 0; j < b_blocks; ++j)
              bulk_load(dst + kSfbOffset + j * kSfBytes,
                        sfb_src + (static_cast<int64_t>(j) * p.atom_cols + ks * kChunksPerStage) * 512,
                        sf_bytes, bar);
            if (!resident) {
              tma_load_2d(dst + kAOffset, a_map, ks * kStageKBytes, t.row0, bar);
              bulk_load(dst + kAOffset + kTileBytes, sfa_src + static_cast<int64_t>(ks) * kSfBytes,
                        sf_bytes, bar);
            }
          }
          __syncwarp();
          ++fills;
          if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
        }
      }
      a_phase ^= 1u;
    }
    if (lane == 0) {
      misc->fills_issued = fills;
      misc->a_fills_issued = a_fills;
    }
  } else if (warp == 1) {
    // ===================================================== MMA issuer
    constexpr uint32_t idesc = make_idesc(kNB * kTileN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t a_phase = 0;
    int it = 0;
    int taken = 0, a_taken = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const Unit u = decode_unit(p, unit);
      for (int nt = u.n_begin; nt < u.n_end && ok; ++nt, ++it) {
        const int acc = it & 1;
        ok = mbar_wait(smem_u32(&misc->acc_empty[acc]), ((it >> 1) & 1u) ^ 1u, abort_flag, kStatusMmaTimeout);
        if (ok && kNB == 2 && it > 0)  // the previous tile's accumulator overlaps this one
          ok = mbar_wait(smem_u32(&misc->shared_cols_free), (it - 1) & 1u, abort_flag, kStatusMmaTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (kNB == 1 ? kTileN : kWideAcc1Col);
        for (int ks = 0; ks < p.k_stages; ++ks) {
          ok = mbar_wait(smem_u32(&misc->full[stage]), phase, abort_flag, kStatusMmaTimeout);
          if (ok) ++taken;
          if (ok && resident && nt == u.n_begin) {
            ok = mbar_wait(smem_u32(&misc->a_full[ks]), a_phase, abort_flag, kStatusMmaTimeout);
            if (ok) ++a_taken;
          }
          if (!ok) break;
          tc_fence_after();
          const int chunks = min(kChunksPerStage, p.atom_cols - ks * kChunksPerStage);
          const uint32_t b_smem = ring_base + stage * ring_stride;
          const uint32_t a_smem = resident ? smem_base + ks * kSlotBytes : b_smem + kAOffset;
          const uint32_t sfa_t = tmem_base + (kNB == 1 ? kSfCol + stage * 32 : kWideSfCol);
          const uint32_t sfb_t = sfa_t + 16;
          const uint64_t a_desc = desc_sw128(a_smem);
          const uint64_t b_desc = desc_sw128(b_smem);
          const uint64_t sfa_desc = desc_sf_atom(a_smem + kTileBytes);
          const uint64_t sfb_desc = desc_sf_atom(b_smem + kSfbOffset);
          if (elect_one()) {
            // The scale-factor atoms of a 64-element chunk go from shared memory to TMEM right
            // before its MMA; copies and MMAs of one thread run in issue order, so a TMEM slot
            // is never overwritten while an earlier MMA still reads it.
            // 64 FP4 values = 32 bytes along K: +2 in 16-byte descriptor units
            auto copies = [&](int c) {
              tc_copy_sf(sfa_t + c * 4, sfa_desc + c * (512 >> 4));
#pragma unroll
              for (int j = 0; j < kNB; ++j)
                tc_copy_sf(sfb_t + (c * kNB + j) * 4, sfb_desc + j * (kSfBytes >> 4) + c * (512 >> 4));
            };
            auto mma = [&](int c) {
              tc_mma_nvf4(d_tmem, a_desc + 2 * c, b_desc + 2 * c, idesc, sfa_t + c * 4, sfb_t + c * 4 * kNB,
                          (ks > 0 || c > 0) ? 1u : 0u);
            };
            if (chunks == kChunksPerStage) {
#pragma unroll
              for (int c = 0; c < kChunksPerStage; ++c) { copies(c); mma(c); }
            } else {
              for (int c = 0; c < chunks; ++c) { copies(c); mma(c); }
            }
            tc_commit(smem_u32(&misc->empty[stage]));
            if (resident && nt == u.n_end - 1) tc_commit(smem_u32(&misc->a_empty[ks]));
          }
          __syncwarp();
          if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&misc->acc_full[acc]));
        __syncwarp();
      }
      a_phase ^= 1u;
    }
    if (lane == 0) {
      misc->fills_taken = taken;
      misc->a_fills_taken = a_taken;
    }
  } else if (warp >= kFirstEpilogueWarp) {
    // ===================================================== epilogue
    // Two groups of four warps.  The unit of work is a 64-column slice of an accumulator:
    // 128-column tiles: group g drains accumulator g (every other tile), slices 0 and 1;
    // 256-column tiles: both groups work on every tile (`drain_tile` has the split).
    const int group = (warp - kFirstEpilogueWarp) >> 2;
    DrainContext ctx;
    ctx.group = group;
    ctx.quarter = warp & 3;  // TMEM lanes this warp may read
    ctx.lane = lane;
    ctx.lane_base = tmem_base + (static_cast<uint32_t>(ctx.quarter * 32) << 16);
    ctx.warp_store = store_base + (warp - kFirstEpilogueWarp) * kStoreBytesPerWarp;
    ctx.out_map = &tmap_out;
    ctx.return_maps = &tmap_return;
    ctx.bar_shared_cols = smem_u32(&misc->shared_cols_free);
    ctx.remote = false;
    ctx.acc1_col = kWideAcc1Col;
    ctx.inv_h = kOut == LM_OUT_NVFP4 ? __ldg(p.out_scale + 1) : 0.0f;
    TileWalker walker;
    int it = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const Unit u = decode_unit(p, unit);
      const RowTile t = walker.at(misc, p, u.mt);
      ctx.alpha = __ldg(p.alpha + (p.alpha_per_expert ? t.expert : 0));
      for (int nt = u.n_begin; nt < u.n_end; ++nt, ++it) {
        if (kNB == 1 && (it & 1) != group) continue;
        const int acc = it & 1;
        ok = mbar_wait(smem_u32(&misc->acc_full[acc]), (it >> 1) & 1u, abort_flag, kStatusEpilogueTimeout);
        if (!ok) break;
        tc_fence_after();
        ctx.bar_acc_empty = smem_u32(&misc->acc_empty[acc]);
        drain_tile<kOut, kAct, kNB>(p, t, ctx, acc, nt);
      }
    }
    if (kOut == LM_OUT_BF16 && lane == 0) tma_store_wait_all();
  }

  // ---- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A bounded wait ran out.  Before shared memory and TMEM are released, wait (bounded again)
    // for what is still in flight: the loads the producer started and nobody consumed complete
    // on their `full` barriers, and a commit after the last MMA tells when the tensor core is
    // done reading shared memory and writing TMEM.
    constexpr long long kDrainLimit = 200000000ll;  // about 0.1 s per barrier
    if (warp == 0 && lane == 0) {
      for (int f = misc->fills_taken; f < misc->fills_issued; ++f)
        mbar_wait_quiet(smem_u32(&misc->full[f % p.ring_stages]), (f / p.ring_stages) & 1u, kDrainLimit);
      if (resident)
        for (int f = misc->a_fills_taken; f < misc->a_fills_issued; ++f)
          mbar_wait_quiet(smem_u32(&misc->a_full[f % p.k_stages]), (f / p.k_stages) & 1u, kDrainLimit);
    }
    if (warp == 1) {
      if (elect_one()) {
        tc_commit(smem_u32(&misc->drain));
        mbar_wait_quiet(smem_u32(&misc->drain), 0, kDrainLimit);
      }
      __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------- CTA-pair kernel
// Two CTAs of a cluster (adjacent SMs) compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA holds 128 rows of A, 128 of the 256 columns of B and
// the accumulator of its own 128 rows, and the tensor cores of both read B from both shared
// memories.  An SM then ingests 38 KB per K stage for 128 x 256 x 256 multiply-adds instead
// of 54 KB: less of the L2-to-SM traffic that bounds the single-CTA kernel.  The ring holds
// five stages.
//
// Roles per CTA as in gemm_kernel: the leader (cluster rank 0) issues the MMAs of the pair and, in front of each, the tcgen05.cp copies that bring that
// chunk's scale-factor atoms from each CTA's shared memory into its own TMEM.  Barriers:
//   full[s]     leader's: the A, B and scale-factor loads of both CTAs complete on it (the
//               peer's TMA loads name the leader's barrier), so scale factors come through
//               tensor maps here as well (eight-byte elements, boxes of 2 KB per atom row).
//   empty[s], acc_full[a]  local in both CTAs, signalled by multicast tcgen05.commit.
//   acc_empty[a]                    leader's; the sixteen epilogue warps of both CTAs arrive.
//   shared_cols_free                leader's; the eight warps that own the shared slice arrive.
constexpr int kPairStageBytes = 2 * kTileBytes + 3 * kSfBytes;  // B half, SFB x2, A, SFA = 38912
// TMEM of a pair CTA: as for 128 x 256 tiles (`kWideAcc1Col`, `kWideSfCol`).
static_assert(kPairStageBytes % 1024 == 0, "pair ring stages must keep 1024-byte alignment");
// The pair's ring is cut from the raw shared-memory budget, not from 18 KB operand slots: five
// stages fit with either output kind (with BF16 staging they fill the 227 KB exactly).
__host__ __device__ constexpr int pair_ring_stages(int out_kind) {
  return (kSmemLimit - 1024 - kMiscBytes - (out_kind == LM_OUT_BF16 ? kStoreBytes : 0)) / kPairStageBytes;
}
__host__ __device__ constexpr int pair_smem_bytes(int out_kind) {
  return 1024 + kMiscBytes + (out_kind == LM_OUT_BF16 ? kStoreBytes : 0) +
         pair_ring_stages(out_kind) * kPairStageBytes;
}
static_assert(pair_ring_stages(LM_OUT_BF16) >= 4 && pair_ring_stages(LM_OUT_NVFP4) <= kMaxRing, "pair ring");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// The shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// TMA load whose completion is counted on a barrier of the pair's other CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the
// MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}

// The same copy in both CTAs of a pair: each from its own shared memory into its own TMEM.
__device__ __forceinline__ void tc_copy_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc_pair(int n) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (0u << 23) |
         (static_cast<uint32_t>(256 >> 4) << 24);
}

// Row tile of cluster rank `rank` inside the 256-row tile `mt` (prefix table built with 256-row
// tiles).  `valid` may be zero: the expert ends before this CTA's half.
__device__ __forceinline__ RowTile pair_row_tile(const Misc* m, const GemmParams& p, int& expert, int mt,
                                                 int rank) {
  while (expert + 1 < p.experts && m->prefix[expert + 1] <= mt) ++expert;
  const int local = mt - m->prefix[expert];
  const int begin = m->cu[expert];
  const int count = m->cu[expert + 1] - begin;
  RowTile t;
  t.expert = expert;
  t.row0 = begin + local * 2 * kTileM + rank * kTileM;
  t.valid = max(0, min(kTileM, count - local * 2 * kTileM - rank * kTileM));
  t.sf_row = begin / kTileM + expert + local * 2 + rank;
  return t;
}

__device__ __forceinline__ uint32_t a_box_rows(int valid) {
  return valid <= 0 ? 0u : (valid <= 32 ? 32u : (valid <= 64 ? 64u : 128u));
}

template <int kOut, int kAct>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a64,
                 const __grid_constant__ CUtensorMap tmap_a32, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_sfa,
                 const __grid_constant__ CUtensorMap tmap_sfb, const __grid_constant__ ReturnMaps tmap_return,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kRingBytes = pair_ring_stages(kOut) * kPairStageBytes;
  const uint32_t store_base = smem_base + kRingBytes;
  Misc* misc = reinterpret_cast<Misc*>(smem_gen + kRingBytes + (kOut == LM_OUT_BF16 ? kStoreBytes : 0));
  volatile int* abort_flag = &misc->abort_flag;

  // ring stage: [B half tile][B scale factors of both column blocks][A tile][A scale factors]
  constexpr uint32_t kOffB = 0;
  constexpr uint32_t kOffSfb = kTileBytes;
  constexpr uint32_t kOffA = kTileBytes + 2 * kSfBytes;
  constexpr uint32_t kOffSfa = kOffA + kTileBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  // ---- one-time setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxRing; ++s) {
      mbar_init(smem_u32(&misc->full[s]), 1);
      mbar_init(smem_u32(&misc->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&misc->acc_full[s]), 1);
      mbar_init(smem_u32(&misc->acc_empty[s]), 16);
    }
    mbar_init(smem_u32(&misc->shared_cols_free), 2 * kWideSharedOwners);  // both CTAs' owners
    mbar_init(smem_u32(&misc->drain), 1);
    misc->abort_flag = 0;
    misc->fills_issued = misc->fills_taken = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // every tcgen05 instruction of this kernel is a pair (cta_group::2) instruction: warp 1 of
    // both CTAs allocates together and each CTA reads the common base from its own shared memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&misc->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  prefill_pdl_wait_and_release();
  if (p.dense) {
    if (threadIdx.x == 0) {
      misc->cu[0] = 0;
      misc->cu[1] = static_cast<int>(p.rows);
    }
  } else {
    for (int e = threadIdx.x; e <= p.experts; e += kThreads)
      misc->cu[e] = *reinterpret_cast<const volatile int32_t*>(p.m_indptr + e);
  }
  __syncthreads();
  if (warp == 2) {
    // exclusive prefix of 256-row tiles per expert; each lane owns 8 experts
    int local[8];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int e = lane * 8 + i;
      int tiles = 0;
      if (e < p.experts) tiles = (misc->cu[e + 1] - misc->cu[e] + 2 * kTileM - 1) / (2 * kTileM);
      local[i] = sum;
      sum += tiles;
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += t;
    }
    const int base = incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int e = lane * 8 + i;
      if (e < p.experts) misc->prefix[e] = base + local[i];
    }
    if (lane == 31) {
      misc->total_m_tiles = incl;
      misc->prefix[p.experts] = incl;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();

  const uint32_t tmem_base = misc->tmem_base;
  const int total_units = misc->total_m_tiles * p.units_per_mtile;
  const int first_unit = blockIdx.x >> 1;
  const int unit_stride = gridDim.x >> 1;

  if (warp == 0) {
    // ===================================================== TMA producer (both CTAs)
    int cursor = 0, peer_cursor = 0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int fills = 0;
    for (int unit = first_unit; unit < total_units && ok; unit += unit_stride) {
      const Unit u = decode_unit(p, unit);
      const RowTile t = pair_row_tile(misc, p, cursor, u.mt, rank);
      const uint32_t a_rows = a_box_rows(t.valid);
      uint32_t peer_a_bytes = 0;
      if (leader) peer_a_bytes = a_box_rows(pair_row_tile(misc, p, peer_cursor, u.mt, 1).valid) * kStageKBytes;
      const CUtensorMap* a_map = a_rows == 32 ? &tmap_a32 : (a_rows == 64 ? &tmap_a64 : &tmap_a);
      for (int nt = u.n_begin; nt < u.n_end && ok; ++nt) {
        const int b_row = t.expert * p.n + nt * 2 * kTileN + rank * kTileN;
        const int sfb_row = t.expert * p.sfb_atom_rows + nt * 2;
        for (int ks = 0; ks < p.k_stages; ++ks) {
          ok = mbar_wait(smem_u32(&misc->empty[stage]), phase ^ 1u, abort_flag, kStatusProducerTimeout);
          if (!ok) break;
          if (elect_one()) {
            const uint32_t bar = smem_u32(&misc->full[stage]);
            const uint32_t dst = smem_base + stage * kPairStageBytes;
            // every byte of both CTAs is counted on the leader's barrier; a scale-factor box is
            // always whole (columns past K read as zero)
            if (leader) {
              mbar_expect_tx(bar, 2 * (kTileBytes + 2 * kSfBytes) + a_rows * kStageKBytes + (a_rows ? kSfBytes : 0) +
                                      peer_a_bytes + (peer_a_bytes ? kSfBytes : 0));
              tma_load_2d(dst + kOffB, &tmap_b, ks * kStageKBytes, b_row, bar);
              tma_load_2d(dst + kOffSfb, &tmap_sfb, ks * (kSfBytes / 8), sfb_row, bar);
              if (a_rows) {
                tma_load_2d(dst + kOffA, a_map, ks * kStageKBytes, t.row0, bar);
                tma_load_2d(dst + kOffSfa, &tmap_sfa, ks * (kSfBytes / 8), t.sf_row, bar);
              }
            } else {
              const uint32_t leader_bar = map_to_cta(bar, 0);
              tma_load_2d_pair(dst + kOffB, &tmap_b, ks * kStageKBytes, b_row, leader_bar);
              tma_load_2d_pair(dst + kOffSfb, &tmap_sfb, ks * (kSfBytes / 8), sfb_row, leader_bar);
              if (a_rows) {  // a half tile past the expert's rows loads neither A nor its scale factors
                tma_load_2d_pair(dst + kOffA, a_map, ks * kStageKBytes, t.row0, leader_bar);
                tma_load_2d_pair(dst + kOffSfa, &tmap_sfa, ks * (kSfBytes / 8), t.sf_row, leader_bar);
              }
            }
          }
          __syncwarp();
          ++fills;
          if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    if (lane == 0) {
      misc->fills_issued = fills;
    }
  } else if (warp == 1) {
    // ===================================================== MMA issuer (leader only)
    if (leader) {
      constexpr uint32_t idesc = make_idesc_pair(2 * kTileN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      int taken = 0;
      bool ok = true;
      for (int unit = first_unit; unit < total_units && ok; unit += unit_stride) {
        const Unit u = decode_unit(p, unit);
        for (int nt = u.n_begin; nt < u.n_end && ok; ++nt, ++it) {
          const int acc = it & 1;
          ok = mbar_wait(smem_u32(&misc->acc_empty[acc]), ((it >> 1) & 1u) ^ 1u, abort_flag, kStatusMmaTimeout);
          if (ok && it > 0)
            ok = mbar_wait(smem_u32(&misc->shared_cols_free), (it - 1) & 1u, abort_flag, kStatusMmaTimeout);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * kWideAcc1Col;
          for (int ks = 0; ks < p.k_stages; ++ks) {
            ok = mbar_wait(smem_u32(&misc->full[stage]), phase, abort_flag, kStatusMmaTimeout);
            if (!ok) break;
            ++taken;
            tc_fence_after();
            const int chunks = min(kChunksPerStage, p.atom_cols - ks * kChunksPerStage);
            const uint32_t stage_smem = smem_base + stage * kPairStageBytes;
            const uint32_t sfa_t = tmem_base + kWideSfCol;
            const uint32_t sfb_t = sfa_t + 16;
            const uint64_t a_desc = desc_sw128(stage_smem + kOffA);
            const uint64_t b_desc = desc_sw128(stage_smem + kOffB);
            const uint64_t sfa_desc = desc_sf_atom(stage_smem + kOffSfa);
            const uint64_t sfb_desc = desc_sf_atom(stage_smem + kOffSfb);
            if (elect_one()) {
              // the atoms of a 64-element chunk go to TMEM right before its MMA; copies and MMAs
              // of one thread run in issue order, so a slot is never overwritten while in use
              auto copies = [&](int c) {
                tc_copy_sf_pair(sfa_t + c * 4, sfa_desc + c * (512 >> 4));
                tc_copy_sf_pair(sfb_t + c * 8, sfb_desc + c * (512 >> 4));
                tc_copy_sf_pair(sfb_t + c * 8 + 4, sfb_desc + (kSfBytes >> 4) + c * (512 >> 4));
              };
              auto mma = [&](int c) {
                tc_mma_nvf4_pair(d_tmem, a_desc + 2 * c, b_desc + 2 * c, idesc, sfa_t + c * 4, sfb_t + c * 8,
                                 (ks > 0 || c > 0) ? 1u : 0u);
              };
              if (chunks == kChunksPerStage) {
#pragma unroll
                for (int c = 0; c < kChunksPerStage; ++c) { copies(c); mma(c); }
              } else {
                for (int c = 0; c < chunks; ++c) { copies(c); mma(c); }
              }
              tc_commit_pair(smem_u32(&misc->empty[stage]));
            }
            __syncwarp();
            if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          if (elect_one()) tc_commit_pair(smem_u32(&misc->acc_full[acc]));
          __syncwarp();
        }
      }
      if (lane == 0) {
        misc->fills_taken = taken;
      }
    }
  } else if (warp >= kFirstEpilogueWarp) {
    // ===================================================== epilogue (both CTAs, own 128 rows)
    DrainContext ctx;
    ctx.group = (warp - kFirstEpilogueWarp) >> 2;
    ctx.quarter = warp & 3;
    ctx.lane = lane;
    ctx.lane_base = tmem_base + (static_cast<uint32_t>(ctx.quarter * 32) << 16);
    ctx.warp_store = store_base + (warp - kFirstEpilogueWarp) * kStoreBytesPerWarp;
    ctx.out_map = &tmap_out;
    ctx.return_maps = &tmap_return;
    ctx.remote = !leader;
    ctx.acc1_col = kWideAcc1Col;
    const uint32_t cols_bar = smem_u32(&misc->shared_cols_free);
    ctx.bar_shared_cols = leader ? cols_bar : map_to_cta(cols_bar, 0);
    ctx.inv_h = kOut == LM_OUT_NVFP4 ? __ldg(p.out_scale + 1) : 0.0f;
    int cursor = 0;
    int it = 0;
    bool ok = true;
    for (int unit = first_unit; unit < total_units && ok; unit += unit_stride) {
      const Unit u = decode_unit(p, unit);
      const RowTile t = pair_row_tile(misc, p, cursor, u.mt, rank);
      ctx.alpha = __ldg(p.alpha + (p.alpha_per_expert ? t.expert : 0));
      for (int nt = u.n_begin; nt < u.n_end; ++nt, ++it) {
        const int acc = it & 1;
        ok = mbar_wait(smem_u32(&misc->acc_full[acc]), (it >> 1) & 1u, abort_flag, kStatusEpilogueTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t empty_bar = smem_u32(&misc->acc_empty[acc]);
        ctx.bar_acc_empty = leader ? empty_bar : map_to_cta(empty_bar, 0);
        drain_tile<kOut, kAct, 2>(p, t, ctx, acc, nt);
      }
    }
    if (kOut == LM_OUT_BF16 && lane == 0) tma_store_wait_all();
  }

  // ---- teardown: neither CTA leaves while the other may still signal its barriers
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // As in gemm_kernel: the leader waits (bounded) for the stage fills that were started and
    // never consumed -- the loads of both CTAs complete on its barriers -- and for its MMAs.
    // A load the peer started for a stage the leader never announced cannot be waited for by
    // anyone; for that case alone both CTAs also let a fixed two million cycles pass.
    constexpr long long kDrainLimit = 200000000ll;
    if (leader && warp == 0 && lane == 0)
      for (int f = misc->fills_taken; f < misc->fills_issued; ++f)
        mbar_wait_quiet(smem_u32(&misc->full[f % p.ring_stages]), (f / p.ring_stages) & 1u, kDrainLimit);
    if (leader && warp == 1) {
      if (elect_one()) {
        tc_commit_pair(smem_u32(&misc->drain));
        mbar_wait_quiet(smem_u32(&misc->drain), 0, kDrainLimit);
      }
      __syncwarp();
    }
    const long long start = clock64();
    while (clock64() - start < 2000000ll) {
    }
    tc_fence_before();
    __syncthreads();
  }
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

#include "gemm_decode.cuh"

// --------------------------------------------------------------- host side
struct PlanData {
  uint32_t magic;
  int32_t out_kind;
  int32_t activation;
  int32_t grid;
  int32_t n_blocks;  // 128-column blocks per tile: 1 or 2
  int32_t pair;      // 1: CTA pairs compute 256 x 256 tiles
  int32_t use_pdl;   // launch as a programmatic dependent of the previous kernel
  GemmParams params;
  alignas(64) CUtensorMap map_a;
  alignas(64) CUtensorMap map_a64;
  alignas(64) CUtensorMap map_a32;
  alignas(64) CUtensorMap map_b;
  alignas(64) CUtensorMap map_out;
  alignas(64) CUtensorMap map_sfa;  // CTA pairs: scale factors as 2 KB boxes per atom row
  alignas(64) CUtensorMap map_sfb;
  alignas(64) ReturnMaps map_return;
};
static_assert(sizeof(PlanData) <= sizeof(lm_gemm_plan), "plan storage too small");
constexpr uint32_t kPlanMagic = 0x4C4D4750u;

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

// Box rows of at most 256 (the limit of a tensor-map box dimension).
int encode_bytes_2d(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                    uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {inner_bytes, rows};
  cuuint64_t strides[1] = {inner_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageKBytes), box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return LM_OK;
}

// BF16 output as 32-row x 64-column boxes in the 128-byte swizzle of the epilogue's staging.
int encode_out_bf16(CUtensorMap* map, void* base, uint64_t cols, uint64_t rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return LM_OK;
}

// Scale-factor atoms as a matrix of eight-byte words: one row per 128-row atom row
// (`atom_cols` atoms of 512 bytes), boxes of one K stage (2 KB) by `box_rows`.
int encode_sf(CUtensorMap* map, const void* base, uint64_t atom_cols, uint64_t atom_rows, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {atom_cols * 64, atom_rows};
  cuuint64_t strides[1] = {atom_cols * 512};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kSfBytes / 8), box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_INT64, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return LM_OK;
}

// ---- decode-shaped plans
struct DecodePlanData {
  uint32_t magic;
  int32_t out_kind;
  int32_t activation;
  int32_t grid;
  int32_t use_pdl;
  DecodeParams params;
  alignas(64) CUtensorMap map_w;    // weights, 128-row boxes
  alignas(64) CUtensorMap map_w64;  // weights, 64-row boxes (half blocks)
  alignas(64) CUtensorMap map_w32;  // weights, 32-row boxes (quarter blocks)
  alignas(64) CUtensorMap map_t8;   // token rows, boxes of 8 / 16 / 32 / 64
  alignas(64) CUtensorMap map_t16;
  alignas(64) CUtensorMap map_t32;
  alignas(64) CUtensorMap map_t64;
};
static_assert(sizeof(DecodePlanData) <= sizeof(lm_gemm_plan), "plan storage too small");
constexpr uint32_t kDecodePlanMagic = 0x4C4D4444u;

constexpr int kDecSmemPerCta = (233472 - 2 * 1024) / 2;  // two CTAs per SM, 1 KB reserved for each
constexpr int dec_smem_bytes(int ring_stages, int stage_bytes) { return 1024 + ring_stages * stage_bytes + kMiscBytes; }

template <int kOut, int kAct>
int launch_decode(const DecodePlanData& pd, cudaStream_t stream) {
  auto kernel = gemm_decode_kernel<kOut, kAct>;
  static bool configured[kMaxDevices] = {};
  int device = 0;
  LM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    LM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemPerCta));
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(pd.grid);
  config.blockDim = dim3(kDecThreads);
  config.dynamicSmemBytes = dec_smem_bytes(pd.params.ring_stages, pd.params.stage_bytes);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pd.use_pdl ? 1 : 0;
  LM_CUDA(cudaLaunchKernelEx(&config, kernel, pd.map_w, pd.map_w64, pd.map_w32, pd.map_t8, pd.map_t16, pd.map_t32, pd.map_t64,
                             pd.params));
  note_launch();
  return LM_OK;
}

int launch_decode_plan(const DecodePlanData& pd, cudaStream_t stream) {
  if (pd.out_kind == LM_OUT_BF16) return launch_decode<LM_OUT_BF16, LM_ACT_NONE>(pd, stream);
  if (pd.out_kind == LM_OUT_F32) return launch_decode<LM_OUT_F32, LM_ACT_NONE>(pd, stream);
  switch (pd.activation) {
    case LM_ACT_SWIGLU: return launch_decode<LM_OUT_NVFP4, LM_ACT_SWIGLU>(pd, stream);
    case LM_ACT_SWIGLU_OAI: return launch_decode<LM_OUT_NVFP4, LM_ACT_SWIGLU_OAI>(pd, stream);
    case LM_ACT_GEGLU: return launch_decode<LM_OUT_NVFP4, LM_ACT_GEGLU>(pd, stream);
    case LM_ACT_REGLU: return launch_decode<LM_OUT_NVFP4, LM_ACT_REGLU>(pd, stream);
    case LM_ACT_RELU2: return launch_decode<LM_OUT_NVFP4, LM_ACT_RELU2>(pd, stream);
  }
  return set_error(LM_ERR_INVALID, "gemm: unknown activation");
}

// Plan of the decode-shaped kernel.  Common argument checks were made by the caller.
int prepare_decode(const lm_gemm_args* a, int out_atom_cols, lm_gemm_plan* plan) {
  LM_REQUIRE(!a->dense, "gemm: swap_ab serves grouped GEMMs");
  LM_REQUIRE(a->direct_routes >= 0 && a->direct_routes <= 32, "gemm: direct route count must be between 0 and 32");
  LM_REQUIRE(a->direct_routes == 0 || a->rows == a->direct_routes, "gemm: direct routes have one row each");
  LM_REQUIRE(!a->broadcast_a || a->direct_routes > 0, "gemm: broadcast A requires direct routing");
  LM_REQUIRE(!a->weights_ahead || a->use_pdl, "gemm: weights_ahead requires use_pdl");
  DecodePlanData pd{};
  pd.magic = kDecodePlanMagic;
  pd.out_kind = a->out_kind;
  pd.activation = a->activation;
  pd.use_pdl = a->use_pdl ? 1 : 0;
  DecodeParams& p = pd.params;
  p.experts = a->experts;
  p.direct = a->direct_routes > 0 ? 1 : 0;
  p.groups = p.direct ? a->direct_routes : a->experts;
  p.broadcast = a->broadcast_a ? 1 : 0;
  p.prefetch = a->weights_ahead ? 1 : 0;
  p.n = a->n;
  p.n_blocks = (a->n + kTileM - 1) / kTileM;
  p.atom_cols = a->k / 64;
  p.k_stages = (p.atom_cols + kChunksPerStage - 1) / kChunksPerStage;
  p.alpha_per_expert = a->alpha_per_expert;
  // no expert can hold more than `rows` rows: steps of up to 32 rows keep the deeper ring
  p.cap = a->rows <= 32 ? 32 : 64;
  p.stage_bytes = kTileBytes + p.cap * kStageKBytes + 2 * kSfBytes;
  // Two CTAs per SM, each with half the shared memory: twice the threads that issue copies and
  // MMAs per SM (the issue rate of single threads bounds a step with few rows), at the same
  // number of stages in flight per SM.
  p.ring_stages = (kDecSmemPerCta - 1024 - kMiscBytes) / p.stage_bytes;
  if (p.ring_stages > 16) p.ring_stages = 16;
  p.rows = a->rows;
  p.m_indptr = a->m_indptr;
  p.sft = static_cast<const uint8_t*>(a->sfa);
  p.sfw = static_cast<const uint8_t*>(a->sfb);
  p.alpha = a->alpha;
  p.out = a->out;
  p.out_sf = static_cast<uint8_t*>(a->out_sf);
  p.out_scale = a->out_scale;
  p.out_row_ptrs = a->out_row_ptrs;
  p.out_atom_cols = out_atom_cols;
  p.clamp_limit = a->clamp_limit;
  p.sigmoid_alpha = a->sigmoid_alpha;
  p.up_bias = a->up_bias;
  const int sms = sm_count();
  LM_REQUIRE(sms > 0, "gemm: no CUDA device");
  pd.grid = a->max_ctas > 0 ? a->max_ctas : 2 * sms;
  // quarter blocks bound the CTAs that can have work: (rows / cap + groups) row tiles at most
  const int64_t max_quarters = (a->rows / p.cap + p.groups) * static_cast<int64_t>(p.n_blocks) * 4;
  if (pd.grid > max_quarters) pd.grid = static_cast<int>(max_quarters);
  const uint64_t k_bytes = static_cast<uint64_t>(a->k / 2);
  const uint64_t w_rows = static_cast<uint64_t>(a->experts) * a->n;
  int rc = encode_bytes_2d(&pd.map_w, a->b, k_bytes, w_rows, kTileM);
  if (rc != LM_OK) return rc;
  rc = encode_bytes_2d(&pd.map_w64, a->b, k_bytes, w_rows, 64);
  if (rc != LM_OK) return rc;
  rc = encode_bytes_2d(&pd.map_w32, a->b, k_bytes, w_rows, 32);
  if (rc != LM_OK) return rc;
  CUtensorMap* token_maps[4] = {&pd.map_t8, &pd.map_t16, &pd.map_t32, &pd.map_t64};
  for (int i = 0; i < 4; ++i) {
    rc = encode_bytes_2d(token_maps[i], a->a, k_bytes, static_cast<uint64_t>(a->rows), 8u << i);
    if (rc != LM_OK) return rc;
  }
  memcpy(plan, &pd, sizeof(pd));
  return LM_OK;
}

template <int kOut, int kAct, int kNB>
int launch_kernel(const PlanData& pd, cudaStream_t stream) {
  auto kernel = gemm_kernel<kOut, kAct, kNB>;
  // the shared-memory opt-in is a per-device attribute of the function
  static bool configured[kMaxDevices] = {};
  int device = 0;
  LM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    LM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(kOut)));
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(pd.grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem_bytes(kOut);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pd.use_pdl ? 1 : 0;
  LM_CUDA(cudaLaunchKernelEx(&config, kernel, pd.map_a, pd.map_a64, pd.map_a32, pd.map_b, pd.map_out,
                             pd.map_return, pd.params));
  note_launch();
  return LM_OK;
}

template <int kOut, int kAct>
int launch_pair(const PlanData& pd, cudaStream_t stream) {
  auto kernel = gemm_pair_kernel<kOut, kAct>;
  static bool configured[kMaxDevices] = {};
  int device = 0;
  LM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    LM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes(kOut)));
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(pd.grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = pair_smem_bytes(kOut);
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pd.use_pdl ? 2 : 1;
  LM_CUDA(cudaLaunchKernelEx(&config, kernel, pd.map_a, pd.map_a64, pd.map_a32, pd.map_b, pd.map_out,
                             pd.map_sfa, pd.map_sfb, pd.map_return, pd.params));
  note_launch();
  return LM_OK;
}

template <int kOut, int kAct>
int launch_variant(const PlanData& pd, cudaStream_t stream) {
  if (pd.pair) return launch_pair<kOut, kAct>(pd, stream);
  return pd.n_blocks == 2 ? launch_kernel<kOut, kAct, 2>(pd, stream) : launch_kernel<kOut, kAct, 1>(pd, stream);
}

int launch_plan(const PlanData& pd, cudaStream_t stream) {
  if (pd.out_kind == LM_OUT_BF16) return launch_variant<LM_OUT_BF16, LM_ACT_NONE>(pd, stream);
  if (pd.out_kind == LM_OUT_F32) return launch_variant<LM_OUT_F32, LM_ACT_NONE>(pd, stream);
  switch (pd.activation) {
    case LM_ACT_SWIGLU: return launch_variant<LM_OUT_NVFP4, LM_ACT_SWIGLU>(pd, stream);
    case LM_ACT_SWIGLU_OAI: return launch_variant<LM_OUT_NVFP4, LM_ACT_SWIGLU_OAI>(pd, stream);
    case LM_ACT_GEGLU: return launch_variant<LM_OUT_NVFP4, LM_ACT_GEGLU>(pd, stream);
    case LM_ACT_REGLU: return launch_variant<LM_OUT_NVFP4, LM_ACT_REGLU>(pd, stream);
    case LM_ACT_RELU2: return launch_variant<LM_OUT_NVFP4, LM_ACT_RELU2>(pd, stream);
  }
  return set_error(LM_ERR_INVALID, "gemm: unknown activation");
}

}  // namespace
}  // namespace lm

extern "C" int lm_gemm_prepare(const lm_gemm_args* a, lm_gemm_plan* plan) {
  using namespace lm;
  LM_REQUIRE(a && plan, "gemm: null argument");
  LM_REQUIRE(a->experts > 0 && a->experts <= kMaxExperts, "gemm: 1..256 experts");
  LM_REQUIRE(a->n > 0 && a->k > 0 && a->k % 64 == 0, "gemm: K must be a positive multiple of 64");
  LM_REQUIRE(a->rows > 0 && a->rows < (1ll << 31), "gemm: rows out of range");
  LM_REQUIRE(a->a && a->b && a->out && a->sfa && a->sfb && a->alpha, "gemm: null operand");
  LM_REQUIRE(a->dense || a->m_indptr, "gemm: grouped GEMM needs m_indptr");
  LM_REQUIRE(!a->dense || a->experts == 1, "gemm: dense GEMM has one group");
  LM_REQUIRE(a->out_kind >= LM_OUT_BF16 && a->out_kind <= LM_OUT_NVFP4, "gemm: unknown output kind");
  LM_REQUIRE((reinterpret_cast<uintptr_t>(a->a) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->b) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a->sfa) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->sfb) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a->out) & 15) == 0,
             "gemm: operands must be 16-byte aligned");
  PlanData pd{};
  pd.magic = kPlanMagic;
  pd.out_kind = a->out_kind;
  pd.activation = a->activation;
  GemmParams& p = pd.params;
  if (a->out_kind == LM_OUT_NVFP4) {
    LM_REQUIRE(a->activation >= LM_ACT_SWIGLU && a->activation <= LM_ACT_RELU2,
               "gemm: NVFP4 output requires an activation");
    LM_REQUIRE(a->n % 128 == 0, "gemm: NVFP4 output requires N aligned to 128");
    LM_REQUIRE(a->out_sf && a->out_scale, "gemm: NVFP4 output needs out_sf and out_scale");
    LM_REQUIRE((reinterpret_cast<uintptr_t>(a->out_sf) & 15) == 0, "gemm: out_sf must be 16-byte aligned");
    const int out_n = a->activation == LM_ACT_RELU2 ? a->n : a->n / 2;
    LM_REQUIRE(out_n % 64 == 0, "gemm: NVFP4 output width must be a multiple of 64");
    p.out_atom_cols = out_n / 64;
  } else {
    LM_REQUIRE(a->activation == LM_ACT_NONE, "gemm: activations require NVFP4 output");
    LM_REQUIRE(a->n % 8 == 0, "gemm: N must be a multiple of 8");
  }
  if (a->swap_ab) return prepare_decode(a, p.out_atom_cols, plan);
  LM_REQUIRE(a->direct_routes == 0 && !a->broadcast_a, "gemm: direct routes require swap_ab");
  p.experts = a->experts;
  p.n = a->n;
  // 256-column tiles on request, when N is whole 128-column blocks and more than one of them:
  // an odd block count leaves half of the last tile empty (its loads fall into the next
  // expert's rows or past the tensor, where TMA fills zeros, and nothing of it is stored)
  pd.n_blocks = (a->tile_n == 256 && a->n % 128 == 0 && a->n >= 256) ? 2 : 1;
  // 256 x 256 tiles on CTA pairs when 256-row tiles are asked for as well
  pd.pair = (pd.n_blocks == 2 && a->tile_m == 256) ? 1 : 0;
  pd.use_pdl = a->use_pdl ? 1 : 0;
  p.n_tiles = (a->n + pd.n_blocks * kTileN - 1) / (pd.n_blocks * kTileN);
  p.atom_cols = a->k / 64;
  p.k_stages = (p.atom_cols + kChunksPerStage - 1) / kChunksPerStage;
  p.sfb_atom_rows = (a->n + 127) / 128;
  p.dense = a->dense;
  p.alpha_per_expert = a->alpha_per_expert;
  p.rows = a->rows;
  p.m_indptr = a->m_indptr;
  p.sfa = static_cast<const uint8_t*>(a->sfa);
  p.sfb = static_cast<const uint8_t*>(a->sfb);
  p.alpha = a->alpha;
  p.out = a->out;
  p.out_sf = static_cast<uint8_t*>(a->out_sf);
  p.out_scale = a->out_scale;
  if (a->out_row_ptrs != nullptr) {
    LM_REQUIRE(a->out_kind == LM_OUT_BF16, "gemm: out_row_ptrs requires BF16 output");
    LM_REQUIRE(a->n % 8 == 0, "gemm: out_row_ptrs requires N to be a multiple of 8");
  }
  p.out_row_ptrs = a->out_row_ptrs;
  if (a->out_blocks != nullptr) {
    LM_REQUIRE(a->out_row_ptrs != nullptr, "gemm: out_blocks goes with out_row_ptrs");
    LM_REQUIRE(a->return_bases != nullptr && a->return_world >= 1 && a->return_world <= LM_EP_MAX_RANKS &&
                   a->return_rows > 0,
               "gemm: out_blocks needs the return buffers of 1..8 ranks");
    LM_REQUIRE(a->n >= 64, "gemm: out_blocks requires N of at least 64");
    for (int g = 0; g < a->return_world; ++g) {
      LM_REQUIRE((a->return_bases[g] & 15) == 0, "gemm: return buffers must be 16-byte aligned");
      const int rc = encode_out_bf16(&pd.map_return.rank[g], reinterpret_cast<void*>(a->return_bases[g]),
                                     static_cast<uint64_t>(a->n), static_cast<uint64_t>(a->return_rows));
      if (rc != LM_OK) return rc;
    }
    p.out_blocks = a->out_blocks;
  }
  p.clamp_limit = a->clamp_limit;
  p.sigmoid_alpha = a->sigmoid_alpha;
  p.up_bias = a->up_bias;
  const int sms = sm_count();
  LM_REQUIRE(sms > 0, "gemm: no CUDA device");
  pd.grid = a->max_ctas > 0 ? a->max_ctas : sms;

  // ---- shared-memory plan: keep A resident when the contraction is short enough
  const int slots = data_slots(a->out_kind);
  const int64_t m_tiles_est = (a->rows + kTileM - 1) / kTileM + (a->dense ? 0 : a->experts / 2);
  // Resident A halves the bytes an SM has to pull in per tile, but the ring that is left must
  // still hold enough bytes in flight to cover the load latency (measured: a 4-stage ring of B
  // tiles loses more than the halved traffic wins), so it needs at least six ring stages.
  p.a_resident =
      (pd.n_blocks == 1 && p.k_stages <= kMaxResident && slots - p.k_stages >= 6 && p.n_tiles >= 2) ? 1 : 0;
  const int row_tile = pd.pair ? 2 * kTileM : kTileM;
  if (p.a_resident) {
    p.ring_stages = slots - p.k_stages < kMaxRing ? slots - p.k_stages : kMaxRing;
    // the longest run of column tiles that still leaves about eight units per CTA
    int run = p.n_tiles;
    while (run > 1 && m_tiles_est * ((p.n_tiles + run - 1) / run) < 8ll * pd.grid) run = (run + 1) / 2;
    p.n_per_unit = run;
  } else {
    const int per_stage = pd.n_blocks + 1;  // B tile(s) and the A tile
    p.ring_stages = slots / per_stage < kMaxRing ? slots / per_stage : kMaxRing;
    if (pd.pair) p.ring_stages = pair_ring_stages(a->out_kind);
    p.n_per_unit = 1;
  }
  p.units_per_mtile = (p.n_tiles + p.n_per_unit - 1) / p.n_per_unit;
  // more CTAs than units would only idle: rows/128 + experts bounds the row tiles
  const int64_t max_units = ((a->rows + row_tile - 1) / row_tile + a->experts) * p.units_per_mtile;
  if (pd.pair) {
    // one cluster of two CTAs per unit in flight
    if (pd.grid > 2 * max_units) pd.grid = static_cast<int>(2 * max_units);
    pd.grid &= ~1;
    LM_REQUIRE(pd.grid >= 2, "gemm: CTA pairs need at least two CTAs");
  } else if (pd.grid > max_units) {
    pd.grid = static_cast<int>(max_units);
  }
  int rc = encode_bytes_2d(&pd.map_a, a->a, static_cast<uint64_t>(a->k / 2), static_cast<uint64_t>(a->rows), kTileM);
  if (rc != LM_OK) return rc;
  rc = encode_bytes_2d(&pd.map_a64, a->a, static_cast<uint64_t>(a->k / 2), static_cast<uint64_t>(a->rows), 64);
  if (rc != LM_OK) return rc;
  rc = encode_bytes_2d(&pd.map_a32, a->a, static_cast<uint64_t>(a->k / 2), static_cast<uint64_t>(a->rows), 32);
  if (rc != LM_OK) return rc;
  rc = encode_bytes_2d(&pd.map_b, a->b, static_cast<uint64_t>(a->k / 2),
                       static_cast<uint64_t>(a->experts) * a->n, pd.pair ? kTileN : pd.n_blocks * kTileN);
  if (rc != LM_OK) return rc;
  // whole 32-row blocks of a BF16 result leave through TMA stores (the SM's plain store path
  // was the bottleneck of short-K GEMMs); rows through a pointer table cannot
  p.tma_store = (a->out_kind == LM_OUT_BF16 && a->out_row_ptrs == nullptr && a->n >= 64) ? 1 : 0;
  p.uneven = p.k_stages >= 6 ? 1 : 0;  // K >= 1536: the main loop of a tile outlasts a three-slice drain
  if (p.tma_store) {
    rc = encode_out_bf16(&pd.map_out, a->out, static_cast<uint64_t>(a->n), static_cast<uint64_t>(a->rows));
    if (rc != LM_OK) return rc;
  }
  if (pd.pair) {
    // A's atom rows: every expert starts a new one (rows / 128 + experts bounds them)
    const uint64_t a_atom_rows =
        a->dense ? static_cast<uint64_t>((a->rows + kTileM - 1) / kTileM)
                 : static_cast<uint64_t>(a->rows / kTileM + a->experts);
    rc = encode_sf(&pd.map_sfa, a->sfa, static_cast<uint64_t>(p.atom_cols), a_atom_rows, 1);
    if (rc != LM_OK) return rc;
    rc = encode_sf(&pd.map_sfb, a->sfb, static_cast<uint64_t>(p.atom_cols),
                   static_cast<uint64_t>(a->experts) * p.sfb_atom_rows, 2);
    if (rc != LM_OK) return rc;
  }
  memcpy(plan, &pd, sizeof(pd));
  return LM_OK;
}

extern "C" int lm_gemm_launch(const lm_gemm_plan* plan, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(plan, "gemm: null plan");
  uint32_t magic;
  memcpy(&magic, plan, sizeof(magic));
  if (magic == kDecodePlanMagic) {
    DecodePlanData dp;  // the caller's storage need not be 64-byte aligned: work on a copy
    memcpy(&dp, plan, sizeof(dp));
    return launch_decode_plan(dp, as_stream(stream));
  }
  PlanData pd;
  memcpy(&pd, plan, sizeof(pd));
  LM_REQUIRE(pd.magic == kPlanMagic, "gemm: plan was not prepared");
  return launch_plan(pd, as_stream(stream));
}

extern "C" int lm_gemm_plan_info(const lm_gemm_plan* plan, int32_t* kernel, int32_t* grid, int32_t* ring_stages) {
  using namespace lm;
  LM_REQUIRE(plan && kernel && grid && ring_stages, "gemm: null argument");
  uint32_t magic;
  memcpy(&magic, plan, sizeof(magic));
  if (magic == kDecodePlanMagic) {
    DecodePlanData dp;
    memcpy(&dp, plan, sizeof(dp));
    *kernel = 3;
    *grid = dp.grid;
    *ring_stages = dp.params.ring_stages;
    return LM_OK;
  }
  PlanData pd;
  memcpy(&pd, plan, sizeof(pd));
  LM_REQUIRE(pd.magic == kPlanMagic, "gemm: plan was not prepared");
  *kernel = pd.pair ? 2 : (pd.n_blocks == 2 ? 1 : 0);
  *grid = pd.grid;
  *ring_stages = pd.params.ring_stages;
  return LM_OK;
}

extern "C" int lm_device_status(uint32_t* out, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(out, "device_status: null pointer");
  LM_CUDA(cudaStreamSynchronize(as_stream(stream)));
  LM_CUDA(cudaMemcpyFromSymbol(out, g_status, sizeof(uint32_t)));
  uint32_t ep = 0;
  const int rc = ep_status_read(&ep);
  if (rc != LM_OK) return rc;
  *out |= ep;
  return LM_OK;
}

extern "C" int lm_device_status_clear(lm_stream_t stream) {
  using namespace lm;
  const uint32_t zero = 0;
  LM_CUDA(cudaStreamSynchronize(as_stream(stream)));
  LM_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(uint32_t)));
  return ep_status_clear();
}

