// Decode-shaped grouped NVFP4 GEMM: few rows per expert, the weights are the stream.
//
// Included by gemm.cu (inside namespace lm, anonymous namespace) after the PTX glue.
//
// The operands swap places: a 128-row block of the expert's WEIGHTS is the M side of
// tcgen05.mma (M = 128) and the expert's 1..64 token rows are the N side (N = 8, 16, 32 or
// 64), so the accumulator is the transposed output block -- lane = weight row = output column,
// TMEM column = token.  Compared with running such a step on 128 x 128 tiles:
//   * a ring stage is 16 KB of weights + 2 KB of their scale factors + a small token box, so
//     nine (<= 32 rows per expert) or seven stages are in flight per SM instead of five or six;
//   * the epilogue touches N columns per lane instead of 128, and stores each token's piece of
//     the output row as 32 consecutive values per warp;
//   * work is dealt in quarter blocks (32 weight rows): when there are fewer than four whole
//     blocks per SM, every SM takes the same contiguous share of quarters (a partial block
//     loads only its 32-row boxes; the rest of the 128-row operand keeps stale bytes whose
//     lanes are never stored), so one token on eight experts keeps all 148 SMs equally busy.
// The contraction runs over the whole K in one accumulator, in the same order as the prefill
// kernels, so decode steps stay bit-identical to prefill steps.
//
// Groups: expert e with rows [m_indptr[e], m_indptr[e+1]) cut into chunks of `cap` rows (32 or
// 64), or -- direct routes -- route r with expert id m_indptr[r], one row (row 0 for every
// route with `broadcast`), scale factors of row r in atom row r.
//
// Programmatic dependent launch: a CTA waits for its predecessor (griddepcontrol.wait) before
// it reads anything that kernel wrote, and lets its own dependents start once it is past that
// wait.  With `prefetch` the routing table is older than the predecessor (the second
// projection of a layer): then only the token loads wait, and each producer warp has the
// weights of one ring stage on their way while the predecessor drains.

constexpr int kDecThreads = 256;         // warps 0, 2, 3 TMA producers (2 after the set-up), 1 MMA, 4..7 epilogue
constexpr int kDecFirstEpilogueWarp = 4;
constexpr uint32_t kDecTmemCols = 256;   // two accumulators of 64 columns, four scale-factor slots of 32
constexpr uint32_t kDecAccCols = 64;
constexpr uint32_t kDecSfCol = 128;
constexpr int kDecQuarterBytes = 32 * kStageKBytes;  // 4096: 32 weight rows of one K stage

struct DecodeParams {
  int groups;         // experts, or direct routes
  int experts;        // experts in the weight tensors
  int n;              // weight rows per expert = output columns
  int n_blocks;       // ceil(n / 128)
  int k_stages;
  int atom_cols;      // k / 64
  int alpha_per_expert;
  int cap;            // token rows per chunk at most: 32 or 64
  int ring_stages;
  int stage_bytes;    // 16 KB weights + cap * 128 B tokens + 2 x 2 KB scale factors
  int direct;         // 1: group r is route r of one token, m_indptr[r] its expert
  int broadcast;      // direct: every route reads token row 0
  int prefetch;       // 1: weights of the first ring pass may load before griddepcontrol.wait
  int64_t rows;
  const int32_t* m_indptr;
  const uint8_t* sft;  // token scale factors, varlen atoms
  const uint8_t* sfw;  // weight scale factors, (expert, n_blocks, k/64, 512)
  const float* alpha;
  void* out;
  uint8_t* out_sf;
  const float* out_scale;
  const uint64_t* out_row_ptrs;
  int out_atom_cols;
  float clamp_limit;
  float sigmoid_alpha;
  float up_bias;
};

struct DecMisc {
  uint64_t full[16];
  uint64_t empty[16];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  int total_row_tiles;
  int fills_issued;
  int fills_taken;
  int pad;
  int cu[kMaxExperts + 1];
  int prefix[kMaxExperts + 2];
};
static_assert(sizeof(DecMisc) <= kMiscBytes, "decode misc block too large");

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct DecRowTile {
  int expert;
  int row0;        // first token row of the chunk (operand and, plus t, output row)
  int valid;       // token rows of the chunk
  int sf_row;      // atom row of the chunk's scale factors
  int sf_col;      // TMEM column of the chunk's first row inside the atom (row / 32)
  int out_sf_row;  // NVFP4 output: atom row of the group's first row ...
  int out_r0;      // ... and the chunk's first row counted from there
};

// Row tile (token chunk) `mt`; a role visits them in increasing order.
struct DecWalker {
  int group = 0;
  __device__ __forceinline__ DecRowTile at(const DecMisc* m, const DecodeParams& p, int mt) {
    DecRowTile t;
    if (p.direct) {
      t.expert = m->cu[mt];
      t.row0 = p.broadcast ? 0 : mt;
      t.valid = 1;
      t.sf_row = p.broadcast ? 0 : mt;
      t.sf_col = 0;
      t.out_sf_row = mt;
      t.out_r0 = 0;
      // an id outside the weights would read another allocation: such a route computes nothing
      if (t.expert < 0 || t.expert >= p.experts) {
        t.expert = 0;
        t.valid = 0;
      }
      return t;
    }
    if (m->prefix[group + 1] <= mt) {
      // the last group whose first row tile is not past mt (empty groups share their
      // successor's value and are skipped): a binary search, since a step with one token
      // leaves hundreds of experts empty
      int lo = group + 1, hi = p.groups;  // prefix[lo] <= mt < prefix[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (m->prefix[mid] <= mt) lo = mid; else hi = mid;
      }
      group = lo;
    }
    const int local = (mt - m->prefix[group]) * p.cap;
    const int begin = m->cu[group];
    const int count = m->cu[group + 1] - begin;
    t.expert = group;
    t.row0 = begin + local;
    t.valid = min(p.cap, count - local);
    t.sf_row = begin / kTileM + group + local / kTileM;
    t.sf_col = (local % kTileM) >> 5;
    t.out_sf_row = begin / kTileM + group;
    t.out_r0 = local;
    return t;
  }
};

// Token rows the MMA covers for a chunk of `valid` rows.
__device__ __forceinline__ int dec_box_rows(int valid) {
  return valid <= 8 ? 8 : (valid <= 16 ? 16 : (valid <= 32 ? 32 : 64));
}

// The share of quarter blocks of one CTA and the walk over it in tiles: a tile is the run of
// quarters [qa, qb) of one (row tile, weight block) unit.
struct DecCursor {
  long long q, q_end;
  __device__ __forceinline__ void init(int total_units, int cta, int ctas) {
    const long long granule = total_units >= 4 * ctas ? 4 : 1;
    const long long items = 4ll * total_units / granule;
    q = items * cta / ctas * granule;
    q_end = items * (cta + 1) / ctas * granule;
  }
  __device__ __forceinline__ bool done() const { return q >= q_end; }
  __device__ __forceinline__ void next(int& unit, int& qa, int& qb) {
    unit = static_cast<int>(q >> 2);
    qa = static_cast<int>(q & 3);
    const long long left = q_end - q;
    qb = left < 4 - qa ? qa + static_cast<int>(left) : 4;
    q += qb - qa;
  }
};

// One ring-stage fill: K stage `ks` of a tile.
struct DecFill {
  DecRowTile t;
  int nb, qa, qb, ks, box;
  uint32_t sf_bytes;
};
struct DecFillIter {
  DecCursor cursor;
  DecWalker walker;
  DecRowTile t;
  int nb = 0, qa = 0, qb = 0, ks = -1;
  __device__ __forceinline__ void init(int total_units, int cta, int ctas) { cursor.init(total_units, cta, ctas); }
  __device__ __forceinline__ bool next(const DecMisc* m, const DecodeParams& p, DecFill& f) {
    if (ks < 0 || ks + 1 == p.k_stages) {
      if (cursor.done()) return false;
      int unit;
      cursor.next(unit, qa, qb);
      const int mt = unit / p.n_blocks;
      nb = unit - mt * p.n_blocks;
      t = walker.at(m, p, mt);
      ks = 0;
    } else {
      ++ks;
    }
    f.t = t;
    f.nb = nb;
    f.qa = qa;
    f.qb = qb;
    f.ks = ks;
    f.box = dec_box_rows(t.valid);
    f.sf_bytes = min(kChunksPerStage, p.atom_cols - ks * kChunksPerStage) * 512;
    return true;
  }
};

__device__ __forceinline__ void tc_load8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld8(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}

// Epilogue of one token: lane = one weight row = one accumulator value `v` (already times alpha).
// Gated: lanes (2j, 2j+1) hold (gate_j, up_j); the warp's 32 lanes make 16 outputs = one
// scale-factor group: 8 bytes of codes (lanes 0 and 16 store a word each) and one factor.
// Unary: the warp's 32 lanes are 32 outputs = two groups.  Same arithmetic, value for value,
// as requant16 of the prefill epilogue.
template <int kAct>
__device__ __forceinline__ void dec_store_nvfp4(const DecodeParams& p, float v, int lane, float inv_h,
                                                uint8_t* codes_row, uint8_t* sf_byte, bool ok) {
  constexpr uint32_t kAll = 0xFFFFFFFFu;
  if (kAct != LM_ACT_RELU2) {
    const float other = __shfl_xor_sync(kAll, v, 1);
    const float h = (lane & 1) ? 0.0f : gated_value<kAct>(v, other, p.clamp_limit, p.sigmoid_alpha, p.up_bias);
    float amax = fabsf(h);
#pragma unroll
    for (int d = 16; d >= 2; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kAll, amax, d));
    const float scaled = amax * (inv_h * inv6());
    const uint32_t sf = f32_to_e4m3(scaled);
    float rescale;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rescale) : "f"(e4m3_to_f32(sf)));
    rescale = fminf(rescale * inv_h, kFltMax);
    const float s = h * rescale;
    const float s_next = __shfl_down_sync(kAll, s, 2);
    uint32_t byte = f32x2_to_e2m1(s, s_next);  // meaningful in lanes 0, 4, 8, ...
    uint32_t word = byte;
    word |= __shfl_down_sync(kAll, byte, 4) << 8;
    word |= __shfl_down_sync(kAll, byte, 8) << 16;
    word |= __shfl_down_sync(kAll, byte, 12) << 24;
    if (ok && (lane & 15) == 0) *reinterpret_cast<uint32_t*>(codes_row + (lane >> 4) * 4) = word;
    if (ok && lane == 0) *sf_byte = static_cast<uint8_t>(sf);
  } else {
    const float x = fmaxf(v, 0.0f);
    const float h = x * x;
    float amax = h;
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kAll, amax, d));
    const float scaled = amax * (inv_h * inv6());
    const uint32_t sf = f32_to_e4m3(scaled);
    float rescale;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rescale) : "f"(e4m3_to_f32(sf)));
    rescale = fminf(rescale * inv_h, kFltMax);
    const float s = h * rescale;
    const float s_next = __shfl_down_sync(kAll, s, 1);
    uint32_t byte = f32x2_to_e2m1(s, s_next);  // meaningful in even lanes
    uint32_t word = byte;
    word |= __shfl_down_sync(kAll, byte, 2) << 8;
    word |= __shfl_down_sync(kAll, byte, 4) << 16;
    word |= __shfl_down_sync(kAll, byte, 6) << 24;
    if (ok && (lane & 7) == 0) *reinterpret_cast<uint32_t*>(codes_row + (lane >> 3) * 4) = word;
    if (ok && (lane & 15) == 0) sf_byte[lane >> 4] = static_cast<uint8_t>(sf);
  }
}

template <int kOut, int kAct>
__global__ void __launch_bounds__(kDecThreads, 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w64,
                   const __grid_constant__ CUtensorMap tmap_w32,
                   const __grid_constant__ CUtensorMap tmap_t8, const __grid_constant__ CUtensorMap tmap_t16,
                   const __grid_constant__ CUtensorMap tmap_t32, const __grid_constant__ CUtensorMap tmap_t64,
                   const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  DecMisc* misc = reinterpret_cast<DecMisc*>(smem_gen + p.ring_stages * p.stage_bytes);
  volatile int* abort_flag = &misc->abort_flag;
  // ring stage: [weights 16 KB][tokens cap x 128 B][weight scale factors 2 KB][token scale factors 2 KB]
  const uint32_t off_tok = kTileBytes;
  const uint32_t off_sfw = kTileBytes + p.cap * kStageKBytes;
  const uint32_t off_sft = off_sfw + kSfBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // One barrier per thread: a single thread initialising all 37 costs most of a microsecond,
  // which counts in a step of a few dozen.
  if (warp >= kDecFirstEpilogueWarp) {
    const int t = threadIdx.x - 32 * kDecFirstEpilogueWarp;
    if (t < 16) mbar_init(smem_u32(&misc->full[t]), 1);
    else if (t < 32) mbar_init(smem_u32(&misc->empty[t - 16]), 1);
    else if (t < 34) mbar_init(smem_u32(&misc->acc_full[t - 32]), 1);
    else if (t < 36) mbar_init(smem_u32(&misc->acc_empty[t - 34]), 4);
    else if (t == 36) mbar_init(smem_u32(&misc->drain), 1);
    else if (t == 37) {
      misc->abort_flag = 0;
      misc->fills_issued = misc->fills_taken = 0;
    }
    if (t < 37) {
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
  }
  if (warp == 0 && lane < 3) {
    // the descriptors the first copies need, fetched while the set-up runs
    const CUtensorMap* map = lane == 0 ? &tmap_w : (lane == 1 ? &tmap_t8 : &tmap_w32);
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&misc->tmem_base)),
                 "r"(kDecTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // The routing table comes from an earlier kernel.  With `prefetch` it was complete before
  // this one's predecessor began (the predecessor waited for it, or was launched the plain way
  // after it), so the table is read at once and only the token operand waits (in the producer
  // warps); otherwise everything waits here.
  // Dependents may start once this CTA is past its wait, not earlier: a dependent that
  // prefetches trusts that everything older than THIS kernel is complete, which holds once
  // every CTA of this kernel has waited for its own predecessor.
  if (!p.prefetch) {
    pdl_wait();
    pdl_launch_dependents();
  }
  const int table = p.direct ? p.groups : p.groups + 1;
  // (a volatile load: one the compiler knows as invariant could move above the wait)
  for (int e = threadIdx.x; e < table; e += kDecThreads)
    misc->cu[e] = *reinterpret_cast<const volatile int32_t*>(p.m_indptr + e);
  __syncthreads();
  if (warp == 2) {
    if (p.direct) {
      if (lane == 0) misc->total_row_tiles = p.groups;
    } else {
      // exclusive prefix of token chunks per expert; each lane owns 8 experts
      int local[8];
      int sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;
        int tiles = 0;
        if (e < p.groups) tiles = (misc->cu[e + 1] - misc->cu[e] + p.cap - 1) / p.cap;
        local[i] = sum;
        sum += tiles;
      }
      int incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += t;
      }
      const int base = incl - sum;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;
        if (e < p.groups) misc->prefix[e] = base + local[i];
      }
      if (lane == 31) {
        misc->total_row_tiles = incl;
        misc->prefix[p.groups] = incl;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = misc->tmem_base;
  const int total_units = misc->total_row_tiles * p.n_blocks;

  if (warp == 0 || warp == 2 || warp == 3) {
    // ===================================================== TMA producers
    // Three warps take the ring-stage fills in turn.  One thread needs 700-900 cycles to wait
    // for a free stage and start the four or five bulk copies of a 16 KB stage (each of these
    // instructions takes on the order of a hundred cycles to issue), which bounded the whole
    // kernel when a single warp did it; the MMA warp needs about 400 cycles per stage.
    const int me = warp == 0 ? 0 : warp - 1;  // 0, 1, 2
    DecFillIter iter;
    iter.init(total_units, blockIdx.x, gridDim.x);
    DecFill f;
    int stage = 0;
    uint32_t phase = 0;
    int fills = 0;
    bool ok = true;
    // With `prefetch` the token operand is the predecessor kernel's output while the weights
    // (and the routing table) are older: each producer starts the weights of its first stage,
    // then waits for the predecessor, then loads the token rows.
    bool waited = p.prefetch == 0;
    while (ok && iter.next(misc, p, f)) {
      if (fills % 3 == me) {
        ok = mbar_wait(smem_u32(&misc->empty[stage]), phase ^ 1u, abort_flag, kStatusProducerTimeout);
        if (!ok) break;
        const uint32_t dst = smem_base + stage * p.stage_bytes;
        const uint32_t bar = smem_u32(&misc->full[stage]);
        if (elect_one()) {
          mbar_expect_tx(bar, (f.qb - f.qa) * kDecQuarterBytes + 2 * f.sf_bytes + f.box * kStageKBytes);
          const int w_row = f.t.expert * p.n + f.nb * kTileM;
          if (f.qa == 0 && f.qb == 4) {
            tma_load_2d(dst, &tmap_w, f.ks * kStageKBytes, w_row, bar);
          } else {
            // a partial block in at most two boxes: 64 rows where a half block is whole
            int q = f.qa;
            while (q < f.qb) {
              if ((q & 1) == 0 && q + 2 <= f.qb) {
                tma_load_2d(dst + q * kDecQuarterBytes, &tmap_w64, f.ks * kStageKBytes, w_row + 32 * q, bar);
                q += 2;
              } else {
                tma_load_2d(dst + q * kDecQuarterBytes, &tmap_w32, f.ks * kStageKBytes, w_row + 32 * q, bar);
                q += 1;
              }
            }
          }
          bulk_load(dst + off_sfw,
                    p.sfw + (static_cast<int64_t>(f.t.expert * p.n_blocks + f.nb) * p.atom_cols +
                             f.ks * kChunksPerStage) * 512,
                    f.sf_bytes, bar);
        }
        __syncwarp();
        if (!waited) {
          pdl_wait();
          pdl_launch_dependents();
          waited = true;
        }
        if (elect_one()) {
          const CUtensorMap* map =
              f.box == 8 ? &tmap_t8 : (f.box == 16 ? &tmap_t16 : (f.box == 32 ? &tmap_t32 : &tmap_t64));
          tma_load_2d(dst + off_tok, map, f.ks * kStageKBytes, f.t.row0, bar);
          bulk_load(dst + off_sft,
                    p.sft + (static_cast<int64_t>(f.t.sf_row) * p.atom_cols + f.ks * kChunksPerStage) * 512,
                    f.sf_bytes, bar);
        }
        __syncwarp();
      }
      ++fills;
      if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
    }
    // (the abort path waits for the stages up to the last one any producer started)
    if (lane == 0) atomicMax(&misc->fills_issued, fills);
  } else if (warp == 1) {
    // ===================================================== MMA issuer
    DecWalker walker;
    DecCursor cursor;
    cursor.init(total_units, blockIdx.x, gridDim.x);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t slot = 0;
    int it = 0;
    int taken = 0;
    bool ok = true;
    while (!cursor.done() && ok) {
      int unit, qa, qb;
      cursor.next(unit, qa, qb);
      const DecRowTile t = walker.at(misc, p, unit / p.n_blocks);
      const uint32_t idesc = make_idesc(dec_box_rows(t.valid));
      const int acc = it & 1;
      ok = mbar_wait(smem_u32(&misc->acc_empty[acc]), ((it >> 1) & 1u) ^ 1u, abort_flag, kStatusMmaTimeout);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kDecAccCols;
      for (int ks = 0; ks < p.k_stages; ++ks) {
        ok = mbar_wait(smem_u32(&misc->full[stage]), phase, abort_flag, kStatusMmaTimeout);
        if (!ok) break;
        ++taken;
        tc_fence_after();
        const int chunks = min(kChunksPerStage, p.atom_cols - ks * kChunksPerStage);
        const uint32_t base = smem_base + stage * p.stage_bytes;
        const uint32_t sfw_t = tmem_base + kDecSfCol + slot * 32;
        const uint32_t sft_t = sfw_t + 16;
        slot = (slot + 1) & 3u;
        const uint64_t w_desc = desc_sw128(base);
        const uint64_t t_desc = desc_sw128(base + off_tok);
        const uint64_t sfw_desc = desc_sf_atom(base + off_sfw);
        const uint64_t sft_desc = desc_sf_atom(base + off_sft);
        if (elect_one()) {
          // the weights take the A (M = 128) side, the tokens the B (N) side; the token chunk's
          // factors start `sf_col` columns into their atom
          for (int c = 0; c < chunks; ++c) {
            tc_copy_sf(sfw_t + c * 4, sfw_desc + c * (512 >> 4));
            tc_copy_sf(sft_t + c * 4, sft_desc + c * (512 >> 4));
            tc_mma_nvf4(d_tmem, w_desc + 2 * c, t_desc + 2 * c, idesc, sfw_t + c * 4, sft_t + c * 4 + t.sf_col,
                        (ks > 0 || c > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&misc->empty[stage]));
        }
        __syncwarp();
        if (++stage == p.ring_stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (elect_one()) tc_commit(smem_u32(&misc->acc_full[acc]));
      __syncwarp();
      ++it;
    }
    if (lane == 0) misc->fills_taken = taken;
  } else if (warp >= kDecFirstEpilogueWarp) {
    // ===================================================== epilogue: warp = lane quarter = 32 weight rows
    const int quarter = warp & 3;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float inv_h = kOut == LM_OUT_NVFP4 ? __ldg(p.out_scale + 1) : 0.0f;
    (void)inv_h;
    DecWalker walker;
    DecCursor cursor;
    cursor.init(total_units, blockIdx.x, gridDim.x);
    int it = 0;
    bool ok = true;
    while (!cursor.done() && ok) {
      int unit, qa, qb;
      cursor.next(unit, qa, qb);
      const int mt = unit / p.n_blocks;
      const int nb = unit - mt * p.n_blocks;
      const DecRowTile t = walker.at(misc, p, mt);
      const int acc = it & 1;
      ok = mbar_wait(smem_u32(&misc->acc_full[acc]), (it >> 1) & 1u, abort_flag, kStatusEpilogueTimeout);
      if (!ok) break;
      tc_fence_after();
      const bool mine = quarter >= qa && quarter < qb;  // this warp's 32 weight rows were computed
      const int col = nb * kTileM + quarter * 32 + lane;  // output column of this lane
      const bool col_ok = mine && col < p.n;
      const float alpha = __ldg(p.alpha + (p.alpha_per_expert ? t.expert : 0));
      const uint32_t taddr = lane_base + acc * kDecAccCols;
      for (int c0 = 0; c0 < t.valid; c0 += 8) {
        uint32_t v[8];
        if (mine) {
          tc_load8(taddr + c0, v);
          tc_wait_ld8(v);
        }
        if (c0 + 8 >= t.valid) {
          // the last columns this warp needs are in registers: hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&misc->acc_empty[acc]));
        }
        if (!mine) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (c0 + j >= t.valid) break;
          const float value = __uint_as_float(v[j]) * alpha;
          const int64_t out_row = static_cast<int64_t>(t.row0) + c0 + j;
          if (kOut == LM_OUT_NVFP4) {
            const int out_n = p.out_atom_cols * 64;
            const int local_row = t.out_r0 + c0 + j;
            const int64_t atom_row = t.out_sf_row + local_row / kTileM;
            const int r = local_row % kTileM;
            // outputs of this warp: gated 16 (one factor), unary 32 (two factors)
            const int out_col0 = kAct == LM_ACT_RELU2 ? nb * kTileM + quarter * 32 : nb * 64 + quarter * 16;
            const int64_t direct_row = p.direct ? mt : out_row;
            uint8_t* codes = static_cast<uint8_t*>(p.out) + direct_row * (out_n >> 1) + (out_col0 >> 1);
            uint8_t* sf_dst = p.out_sf + sf_offset(atom_row, p.out_atom_cols, r, out_col0 >> 4);
            dec_store_nvfp4<kAct>(p, value, lane, inv_h, codes, sf_dst, true);
          } else {
            const int64_t direct_row = p.direct ? mt : out_row;
            if (kOut == LM_OUT_BF16) {
              __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + direct_row * p.n;
              if (p.out_row_ptrs != nullptr)
                dst = reinterpret_cast<__nv_bfloat16*>(__ldg(reinterpret_cast<const unsigned long long*>(p.out_row_ptrs) + direct_row));
              if (col_ok) dst[col] = __float2bfloat16_rn(value);
            } else {
              if (col_ok) static_cast<float*>(p.out)[direct_row * p.n + col] = value;
            }
          }
        }
      }
      if (t.valid <= 0) {
        // nothing to read (a direct route with an id outside the weights): still hand back
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&misc->acc_empty[acc]));
      }
      ++it;
    }
  }

  // ---- teardown (as in gemm_kernel: on abort, wait for what is still in flight)
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    constexpr long long kDrainLimit = 200000000ll;
    if (warp == 0 && lane == 0)
      for (int f = misc->fills_taken; f < misc->fills_issued; ++f)
        mbar_wait_quiet(smem_u32(&misc->full[f % p.ring_stages]), (f / p.ring_stages) & 1u, kDrainLimit);
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDecTmemCols)
                 : "memory");
  }
}
