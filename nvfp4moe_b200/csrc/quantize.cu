// Row-wise BF16/FP32 -> NVFP4 quantization (HBM-bound).
//
// One CTA covers one 128-row scale-factor atom row and 512 features.  A warp
// streams one row slice at a time: each lane owns one 16-element group (32 B of
// BF16), so a warp reads 1 KB contiguous and writes 256 B of packed codes.
// Scale factors are staged in shared memory in atom order and leave the CTA as
// 16-byte stores, so every 512-byte atom is written whole.
#include "common.cuh"
#include "quantize_math.cuh"

namespace lm {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTileRows = 128;
constexpr int kTileCols = 512;  // 32 lanes x 16 elements

struct QuantParams {
  const void* x;
  int64_t rows;
  int features;
  const int32_t* m_indptr;
  int experts;
  int64_t rows_per_group;
  int tiles_per_group;
  const float* scale_pair;
  const int32_t* gather;
  uint8_t* q;
  uint8_t* sf;
  int sf_mode;
  int te_math;
};

template <typename In>
__global__ void __launch_bounds__(kThreads, 4) quantize_rowwise_kernel(QuantParams p) {
  __shared__ __align__(16) uint8_t s_sf[(kTileCols / 64) * 512];
  __shared__ int s_group[4];  // group, local tile, first row, valid rows

  const int tid = threadIdx.x;
  const int64_t atom_row = blockIdx.x;
  const int col0 = blockIdx.y * kTileCols;

  // ---- which rows does this atom row hold?
  if (tid == 0) s_group[3] = 0;
  __syncthreads();
  if (p.sf_mode == LM_SF_VARLEN) {
    for (int e = tid; e < p.experts; e += kThreads) {
      int lo = __ldg(p.m_indptr + e);
      int hi = __ldg(p.m_indptr + e + 1);
      int64_t first = lo / kTileRows + e;
      int64_t next = hi / kTileRows + e + 1;
      if (atom_row >= first && atom_row < next) {
        int lt = static_cast<int>(atom_row - first);
        int remaining = (hi - lo) - lt * kTileRows;
        if (remaining > 0) {
          s_group[0] = e;
          s_group[1] = lt;
          s_group[2] = lo + lt * kTileRows;
          s_group[3] = remaining < kTileRows ? remaining : kTileRows;
        }
      }
    }
  } else if (tid == 0) {
    int64_t group = p.sf_mode == LM_SF_BATCHED ? atom_row / p.tiles_per_group : 0;
    int lt = p.sf_mode == LM_SF_BATCHED ? static_cast<int>(atom_row % p.tiles_per_group)
                                        : static_cast<int>(atom_row);
    int64_t group_rows = p.sf_mode == LM_SF_BATCHED ? p.rows_per_group : p.rows;
    int64_t remaining = group_rows - static_cast<int64_t>(lt) * kTileRows;
    s_group[0] = static_cast<int>(group);
    s_group[1] = lt;
    s_group[2] = 0;
    s_group[3] = remaining <= 0 ? 0 : (remaining < kTileRows ? static_cast<int>(remaining) : kTileRows);
  }
  __syncthreads();
  const int valid = s_group[3];
  if (valid == 0) return;
  int64_t row0;
  if (p.sf_mode == LM_SF_VARLEN) {
    row0 = s_group[2];
  } else {
    row0 = static_cast<int64_t>(s_group[0]) * (p.sf_mode == LM_SF_BATCHED ? p.rows_per_group : 0) +
           static_cast<int64_t>(s_group[1]) * kTileRows;
  }

  const bool blocked = p.sf_mode != LM_SF_LINEAR;
  if (blocked && valid < kTileRows) {
    uint4* z = reinterpret_cast<uint4*>(s_sf);
    for (int i = tid; i < static_cast<int>(sizeof(s_sf) / 16); i += kThreads) z[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }

  const float pts = __ldg(p.scale_pair);
  const float inv_pts = __ldg(p.scale_pair + 1);
  const bool te = p.te_math != 0;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int col = col0 + lane * 16;
  const bool col_ok = col < p.features;
  const In* x = static_cast<const In*>(p.x);
  const int groups_per_row = p.features >> 4;

  // The warp owns rows warp, warp + 8, ...: lane i fetches the source row of the i-th of
  // them up front, so no row load waits on an index load.
  int64_t my_src = 0;
  {
    const int r = warp + lane * kWarps;
    if (lane < kTileRows / kWarps && r < valid) {
      my_src = row0 + r;
      if (p.gather != nullptr) my_src = __ldg(p.gather + my_src);
    }
  }

  constexpr int kUnroll = Slice<In>::kUnroll;
  for (int base = 0; base < kTileRows / kWarps; base += kUnroll) {
    if (warp + base * kWarps >= valid) break;
    Slice<In> v[kUnroll];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = warp + (base + u) * kWarps;
      const int64_t src = __shfl_sync(0xFFFFFFFFu, my_src, base + u);
      ok[u] = col_ok && r < valid;
      if (ok[u]) v[u].load(x + src * p.features + col);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (!ok[u]) continue;
      const int r = warp + (base + u) * kWarps;
      uint2 packed;
      uint32_t sf_byte = quantize_group(v[u], pts, inv_pts, te, &packed);
      int64_t out_row = row0 + r;
      *reinterpret_cast<uint2*>(p.q + out_row * (p.features >> 1) + (col >> 1)) = packed;
      if (blocked) {
        s_sf[(lane >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (lane & 3)] =
            static_cast<uint8_t>(sf_byte);
      } else {
        p.sf[out_row * groups_per_row + (col >> 4)] = static_cast<uint8_t>(sf_byte);
      }
    }
  }
  if (!blocked) return;
  __syncthreads();

  // ---- atoms leave as 16-byte stores: thread i -> atom i / 32, piece i % 32
  const int atom_cols = p.features >> 6;
  const int atom = tid >> 5;
  const int atom_col = (col0 >> 6) + atom;
  if (atom_col < atom_cols) {
    uint4 piece = reinterpret_cast<const uint4*>(s_sf)[tid];
    uint8_t* dst = p.sf + (atom_row * atom_cols + atom_col) * 512 + (tid & 31) * 16;
    *reinterpret_cast<uint4*>(dst) = piece;
  }
}

// ------------------------------------------------- quantize once, scatter to slots
// One warp per token: its destinations (one row per route) are worked out once, then every
// 512-feature slice is quantized once and its packed codes (256 B, one coalesced store) and
// scale factors (eight 4-byte words, one per 64-feature atom) are written to every
// expert-major row the token was routed to.
struct ScatterQuantParams {
  const __nv_bfloat16* x;
  int64_t tokens;
  int features;
  int top_k;
  const int32_t* slots;
  const int32_t* topk_ids;
  const int32_t* m_indptr;
  const float* scale_pair;
  uint8_t* q;
  uint8_t* sf;
};

__global__ void __launch_bounds__(kThreads) quantize_scatter_kernel(ScatterQuantParams p) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (token >= p.tokens) return;
  // Destination of route `lane` (lanes beyond top_k idle), computed once per token: the
  // row's packed bytes and the byte of its first scale-factor word (atom column 0).
  const int atom_cols = p.features >> 6;
  uint8_t* my_q = nullptr;
  uint8_t* my_sf = nullptr;
  if (lane < p.top_k) {
    const int slot = __ldg(p.slots + token * p.top_k + lane);
    if (slot >= 0) {
      const int e = __ldg(p.topk_ids + token * p.top_k + lane);
      const int lo = __ldg(p.m_indptr + e);
      const int local = slot - lo;
      const int atom_row = lo / kTileRows + e + local / kTileRows;
      const int r = local % kTileRows;
      my_q = p.q + static_cast<int64_t>(slot) * (p.features >> 1);
      my_sf = p.sf + static_cast<int64_t>(atom_row) * atom_cols * 512 + (r & 31) * 16 + (r >> 5) * 4;
    }
  }
  const float pts = __ldg(p.scale_pair);
  const float inv_pts = __ldg(p.scale_pair + 1);
  const __nv_bfloat16* x_row = p.x + token * p.features;
  // the warp walks the token's 512-feature slices; the next slice is loaded while this one
  // is quantized and stored
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
    // four neighbouring lanes hold the four factors of one atom word
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
      if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(sf_row + static_cast<int64_t>(col >> 6) * 512) = word;
    }
    cur = next;
  }
}

}  // namespace
}  // namespace lm

extern "C" int lm_quantize_rowwise(const void* x, int x_dtype, int64_t rows, int features,
                                   const int32_t* m_indptr, int experts, int64_t rows_per_group,
                                   const float* scale_pair, const int32_t* gather_idx, uint8_t* q,
                                   uint8_t* sf, int sf_mode, int te_math, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(x && scale_pair && q && sf, "quantize: null pointer");
  LM_REQUIRE(x_dtype == LM_DTYPE_BF16 || x_dtype == LM_DTYPE_F32, "quantize: x must be BF16 or FP32");
  LM_REQUIRE(features > 0 && features % 64 == 0, "quantize: features must be a multiple of 64");
  LM_REQUIRE(rows >= 0, "quantize: negative row count");
  LM_REQUIRE(sf_mode >= LM_SF_VARLEN && sf_mode <= LM_SF_LINEAR, "quantize: unknown sf_mode");
  if (rows == 0) return LM_OK;
  QuantParams p{};
  p.x = x;
  p.rows = rows;
  p.features = features;
  p.m_indptr = m_indptr;
  p.experts = experts;
  p.rows_per_group = rows_per_group;
  p.scale_pair = scale_pair;
  p.gather = gather_idx;
  p.q = q;
  p.sf = sf;
  p.sf_mode = sf_mode;
  p.te_math = te_math;
  int64_t atom_rows;
  if (sf_mode == LM_SF_VARLEN) {
    LM_REQUIRE(m_indptr != nullptr && experts > 0, "quantize: varlen layout needs m_indptr");
    atom_rows = (rows + 127) / 128 + experts;
  } else if (sf_mode == LM_SF_BATCHED) {
    LM_REQUIRE(rows_per_group > 0 && rows % rows_per_group == 0,
               "quantize: rows must be a multiple of rows_per_group");
    p.tiles_per_group = static_cast<int>((rows_per_group + 127) / 128);
    atom_rows = (rows / rows_per_group) * p.tiles_per_group;
  } else {
    atom_rows = (rows + 127) / 128;
  }
  LM_REQUIRE(atom_rows < (1ll << 31), "quantize: too many rows");
  dim3 grid(static_cast<unsigned>(atom_rows), (features + kTileCols - 1) / kTileCols);
  if (x_dtype == LM_DTYPE_BF16) {
    quantize_rowwise_kernel<__nv_bfloat16><<<grid, kThreads, 0, as_stream(stream)>>>(p);
    note_launch();
  } else {
    quantize_rowwise_kernel<float><<<grid, kThreads, 0, as_stream(stream)>>>(p);
    note_launch();
  }
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_quantize_decode(const void* x, int64_t tokens, int features, int top_k,
                                  const int32_t* slots, const int32_t* topk_ids,
                                  const int32_t* m_indptr, int experts, const float* scale_pair,
                                  uint8_t* q, uint8_t* sf, lm_stream_t stream) {
  using namespace lm;
  (void)experts;
  LM_REQUIRE(x && slots && topk_ids && m_indptr && scale_pair && q && sf, "quantize_decode: null pointer");
  LM_REQUIRE(features > 0 && features % 64 == 0, "quantize_decode: features must be a multiple of 64");
  LM_REQUIRE(top_k > 0 && tokens >= 0, "quantize_decode: bad sizes");
  if (tokens == 0) return LM_OK;
  LM_REQUIRE(top_k <= 32, "quantize_decode: top_k must be at most 32");
  ScatterQuantParams p{static_cast<const __nv_bfloat16*>(x), tokens, features, top_k, slots,
                       topk_ids, m_indptr, scale_pair, q, sf};
  dim3 grid(static_cast<unsigned>((tokens + kWarps - 1) / kWarps));
  quantize_scatter_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
