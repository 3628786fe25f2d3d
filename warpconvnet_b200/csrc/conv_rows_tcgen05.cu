// Convolutions in which every output row has exactly ONE (input row, kernel offset) pair, run
// input-stationary on the tensor cores (sm_100a): the 1x1x1 convolution (output row = input row, or
// a permutation of it), and the transposed convolution whose window equals its stride (2x2x2,
// stride 2: every fine voxel has one parent).
//
// Output-stationary, such a layer gathers one 2*C_in-byte row per output row through 16-byte
// requests and uses a 128-row MMA tile for a single offset.  Seen from the INPUT side the layer is
// a plain GEMM over consecutive rows,
//     Y[j, k*C_out : (k+1)*C_out] = X[j, :] @ W[k]        for every input row j and offset k,
// followed by a scatter: row j's k-th block goes to output row dst[k][j] (or nowhere when that
// pair does not exist).  So
//   * the rows of X arrive as 128 x BK tiles through TMA (cp.async.bulk.tensor, hardware swizzle),
//     each row read once per weight chunk instead of once per output row that needs it;
//   * the weights of a chunk of offsets (up to 256 output columns) stay in shared memory across
//     all row tiles a CTA processes; the chunk of the next unit is loaded behind the current one;
//   * accumulators are two to four sets of up to 256 TMEM columns, so the epilogues of the previous
//     tiles (whose latency is a table lookup, a TMEM load and scattered stores) overlap the MMAs of
//     the next ones;
//   * eight epilogue warps read TMEM, apply scale / shift / residual / ReLU and store each
//     C_out-wide block at its destination row.
// Work unit = (chunk of offsets, row tile); units are numbered chunk-major and dealt round-robin to
// a persistent grid, so a CTA changes its weight chunk only a few times on large inputs.
//
// Every wait is bounded (tcgen05_common.cuh); a kernel that gives up sets the status word, drains
// its copies and frees its tensor memory.
#include <cuda.h>

#include "tcgen05_common.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int MAX_STAGES = 24;         // row-tile ring: up to 192 KB in flight per multiprocessor
constexpr int MAX_Q = 8;               // offsets per chunk
constexpr int MAX_ACC = 4;             // accumulator sets in tensor memory
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, EPI_WARP0 = 2, EPI_WARPS = 8;
constexpr int THREADS = (EPI_WARP0 + EPI_WARPS) * 32;
constexpr int MAX_COLS = 256;          // output columns of one chunk (one MMA's N)
constexpr int SMEM_BUDGET = 220 * 1024;

struct RowsParams {
  const char* wpacked;       // packed weights: [K][c_in/BK] swizzled tiles of [c_out][BK]
  const int32_t* dst;        // [K][M_in] destination rows (-1: none), or null: K == 1 and dst = row
  int64_t M_in, num_out;
  int K, c_in, c_out, c_store;  // c_out: packed width (multiple of 16), c_store: columns that exist
  int q, nchunks, nbuf, stages; // offsets per chunk, chunks, weight buffers, row-tile ring depth
  int nacc;                     // accumulator sets (2..4, as many as fit in 512 columns)
  int64_t tiles, units;
  const float* scale;
  const float* shift;
  const void* residual;
  int64_t res_ld;
  int relu;
  void* out;
  int64_t out_ld;
  int vec;                   // bytes every output / residual row start is aligned to: 32, 16, 8 or 0
  int32_t* dev_status;
};

// Ring cursor: slot index and the parity of the phase the slot is in.
struct Ring {
  int slot, phase, depth;
  __device__ __forceinline__ void advance() {
    if (++slot == depth) { slot = 0; phase ^= 1; }
  }
};

struct RowsControl {
  uint64_t a_full[MAX_STAGES], a_empty[MAX_STAGES];
  uint64_t b_full[2], b_empty[2];
  uint64_t acc_full[MAX_ACC], acc_empty[MAX_ACC];
  uint32_t tmem_holder;
  int32_t skip;
  float sc[MAX_COLS], sh[MAX_COLS];
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// 32 bytes in one request: a whole sector per lane, so that rows scattered over the output cost the
// L2 one full-sector write each instead of two half-sector ones.
__device__ __forceinline__ void st_global_32B(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// One 16-column piece of a row: convert and store columns [c0, c0 + 16) that exist (< c_store).
template <typename TO>
__device__ __forceinline__ void store_piece(TO* orow, int c0, const float (&y)[16], int c_store, int vec) {
  constexpr int PER16 = 16 / (int)sizeof(TO), PER8 = 8 / (int)sizeof(TO);
  __align__(32) TO tmp[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) tmp[i] = wcn_from_float<TO>(y[i]);
  const int valid = min(16, c_store - c0);
  if (vec == 32 && valid == 16) {
#pragma unroll
    for (int i = 0; i < (int)sizeof(TO) / 2; ++i)   // 16 columns are 32 (fp16 / bf16) or 64 bytes (fp32)
      st_global_32B(reinterpret_cast<char*>(orow + c0) + 32 * i, reinterpret_cast<const uint32_t*>(tmp) + 8 * i);
  } else if (vec >= 16 && valid == 16) {
#pragma unroll
    for (int i = 0; i < 16 / PER16; ++i) reinterpret_cast<uint4*>(orow + c0)[i] = reinterpret_cast<const uint4*>(tmp)[i];
  } else if (vec >= 8) {
#pragma unroll
    for (int i = 0; i < 16 / PER8; ++i) {
      if ((i + 1) * PER8 <= valid) {
        reinterpret_cast<uint2*>(orow + c0)[i] = reinterpret_cast<const uint2*>(tmp)[i];
      } else {
#pragma unroll
        for (int e = 0; e < PER8; ++e)
          if (i * PER8 + e < valid) orow[c0 + i * PER8 + e] = tmp[i * PER8 + e];
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < valid) orow[c0 + i] = tmp[i];
  }
}

template <typename TO>
__device__ __forceinline__ void add_residual(const TO* rrow, int c0, float (&y)[16], int c_store, int vec) {
  constexpr int PER16 = 16 / (int)sizeof(TO);
  const int valid = min(16, c_store - c0);
  if (vec >= 16 && valid == 16) {
    __align__(16) TO tmp[16];
#pragma unroll
    for (int i = 0; i < 16 / PER16; ++i) reinterpret_cast<uint4*>(tmp)[i] = __ldg(reinterpret_cast<const uint4*>(rrow + c0) + i);
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] += wcn_to_float<TO>(tmp[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < valid) y[i] += wcn_to_float<TO>(rrow[c0 + i]);
  }
}

// Position in the unit sequence of a CTA: units are numbered chunk-major, a CTA takes every
// grid-th one.  Kept as (chunk, tile) and advanced by additions only.
struct UnitCursor {
  int chunk, tile;
  __device__ __forceinline__ void advance(int step, int tiles) {
    tile += step;
    while (tile >= tiles) { tile -= tiles; ++chunk; }
  }
};

template <int BK, bool BF16, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
conv_rows_tcgen05_kernel(const __grid_constant__ CUtensorMap feats_map, const RowsParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int RB = BK * 2;
  constexpr int A_BYTES = BLOCK_M * RB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KB = p.c_in / BK;
  const int B_TILE = p.c_out * RB;          // one (offset, channel slice) weight tile
  const int B_SLICE = p.q * B_TILE;         // the chunk's tiles of one channel slice, stacked along N
  const int B_BUF = KB * B_SLICE;
  const int tiles = (int)p.tiles, grid = (int)gridDim.x;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t b_base = base;
  const uint32_t a_base = b_base + (uint32_t)(p.nbuf * B_BUF);
  RowsControl* ctl = reinterpret_cast<RowsControl*>(gen + p.nbuf * B_BUF + p.stages * A_BYTES);
  auto bar = [](uint64_t* b) { return smem_u32(b); };
  UnitCursor first{0, 0};
  first.advance((int)blockIdx.x, tiles);

  if (tid == 0) ctl->skip = *(volatile int32_t*)p.dev_status;
  __syncthreads();
  if (ctl->skip == (int)WCN_ERR_WAIT_EXPIRED) {
    // A kernel on this status word gave up earlier: compute nothing and mark this launch's rows.
    const TO nan = wcn_from_float<TO>(__int_as_float(0x7FC00000));
    for (UnitCursor c = first; c.chunk < p.nchunks; c.advance(grid, tiles)) {
      const int k0 = c.chunk * p.q, qc = min(p.q, p.K - k0);
      for (int i = tid; i < qc * BLOCK_M; i += THREADS) {
        const int64_t row = (int64_t)c.tile * BLOCK_M + (i % BLOCK_M);
        if (row >= p.M_in) continue;
        const int64_t d = p.dst ? (int64_t)__ldg(&p.dst[(int64_t)(k0 + i / BLOCK_M) * p.M_in + row]) : row;
        if (d < 0 || d >= p.num_out) continue;
        for (int col = 0; col < p.c_store; ++col) reinterpret_cast<TO*>(p.out)[d * p.out_ld + col] = nan;
      }
    }
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(bar(&ctl->a_full[s]), 1); mbar_init(bar(&ctl->a_empty[s]), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(&ctl->b_full[i]), 1);
      mbar_init(bar(&ctl->b_empty[i]), 1);
    }
    for (int i = 0; i < MAX_ACC; ++i) {
      mbar_init(bar(&ctl->acc_full[i]), 1);
      mbar_init(bar(&ctl->acc_empty[i]), EPI_WARPS / 2);   // the four warps that finish a given unit
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&feats_map)) : "memory");
  }
  for (int i = tid; i < p.c_out; i += THREADS) {
    ctl->sc[i] = (p.scale && i < p.c_store) ? __ldg(&p.scale[i]) : 1.f;
    ctl->sh[i] = (p.shift && i < p.c_store) ? __ldg(&p.shift[i]) : 0.f;
  }
  const int ncols = p.q * p.c_out;  // accumulator columns of one set
  uint32_t tmem_total = 32;
  while ((int)tmem_total < p.nacc * ncols) tmem_total <<= 1;
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&ctl->tmem_holder), tmem_total);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_holder;

  bool ok = true;
  if (warp == PRODUCER_WARP) {
    // ================================================================ copies: weights and row tiles
    if (lane == 0) {
      Ring ra{0, 0, p.stages};
      int bbuf = 0, bphase = 0, cur_chunk = -1;
      int issued = 0;  // row-tile copies issued (for the drain below)
      for (UnitCursor c = first; c.chunk < p.nchunks && ok; c.advance(grid, tiles)) {
        if (c.chunk != cur_chunk) {
          if (cur_chunk >= 0 && ++bbuf == p.nbuf) { bbuf = 0; bphase ^= 1; }
          cur_chunk = c.chunk;
          const int k0 = c.chunk * p.q, qc = min(p.q, p.K - k0);
          if (!mbar_wait(bar(&ctl->b_empty[bbuf]), bphase ^ 1, p.dev_status)) { ok = false; break; }
          const uint32_t fullb = bar(&ctl->b_full[bbuf]);
          mbar_expect_tx(fullb, (uint32_t)(KB * qc * B_TILE));
          for (int s = 0; s < KB; ++s)
            for (int o = 0; o < qc; ++o)
              bulk_copy_g2s(b_base + (uint32_t)(bbuf * B_BUF + s * B_SLICE + o * B_TILE),
                            p.wpacked + ((int64_t)(k0 + o) * KB + s) * B_TILE, (uint32_t)B_TILE, fullb);
        }
        const int row0 = c.tile * BLOCK_M;
        for (int s = 0; s < KB; ++s) {
          if (!mbar_wait(bar(&ctl->a_empty[ra.slot]), ra.phase ^ 1, p.dev_status)) { ok = false; break; }
          const uint32_t fullb = bar(&ctl->a_full[ra.slot]);
          mbar_expect_tx(fullb, (uint32_t)A_BYTES);
          tma_load_2d(a_base + (uint32_t)(ra.slot * A_BYTES), &feats_map, s * BK, row0, fullb);
          ra.advance();
          ++issued;
        }
      }
      if (!ok) {
        // gave up: let the copies already issued land before the CTA's shared memory is released
        const int pending = issued < p.stages ? issued : p.stages;
        for (int s = 0; s < pending; ++s)
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(bar(&ctl->a_full[s]), 0) || mbar_try_wait(bar(&ctl->a_full[s]), 1)) break;
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      Ring ra{0, 0, p.stages};
      int bbuf = 0, bphase = 0, cur_chunk = -1, ab = 0, aphase = 0;
      uint32_t idesc = 0;
      const uint64_t adesc0 = smem_desc<RB>(a_base), bdesc0 = smem_desc<RB>(b_base);
      uint64_t bdesc_buf = bdesc0;
      for (UnitCursor c = first; c.chunk < p.nchunks && ok; c.advance(grid, tiles)) {
        if (c.chunk != cur_chunk) {
          if (cur_chunk >= 0) {
            umma_commit(bar(&ctl->b_empty[bbuf]));  // the previous chunk's weights may be overwritten
            if (++bbuf == p.nbuf) { bbuf = 0; bphase ^= 1; }
          }
          cur_chunk = c.chunk;
          const int qc = min(p.q, p.K - c.chunk * p.q);
          idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                  ((uint32_t)((qc * p.c_out) >> 3) << 17) | ((uint32_t)(BLOCK_M >> 4) << 24);
          bdesc_buf = bdesc0 + (uint64_t)((bbuf * B_BUF) >> 4);
          if (!mbar_wait(bar(&ctl->b_full[bbuf]), bphase, p.dev_status)) { ok = false; break; }
        }
        if (!mbar_wait(bar(&ctl->acc_empty[ab]), aphase ^ 1, p.dev_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(ab * ncols);
        for (int s = 0; s < KB; ++s) {
          if (!mbar_wait(bar(&ctl->a_full[ra.slot]), ra.phase, p.dev_status)) { ok = false; break; }
          tc_fence_after();
          // (descriptor start addresses are in 16-byte units: a slot or slice further is a plain addition)
          const uint64_t adesc = adesc0 + (uint64_t)((ra.slot * A_BYTES) >> 4);
          const uint64_t bdesc = bdesc_buf + (uint64_t)((s * B_SLICE) >> 4);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_f16(d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (s | kk) ? 1u : 0u);
          umma_commit(bar(&ctl->a_empty[ra.slot]));
          ra.advance();
        }
        if (!ok) break;
        umma_commit(bar(&ctl->acc_full[ab]));
        if (++ab == p.nacc) { ab = 0; aphase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ================================================================ epilogue (8 warps)
    // TMEM lanes 32*(warp % 4).. belong to this warp.  The two warps of a lane quarter take
    // alternate units: what an epilogue pays per unit besides the data (barrier round trip, table
    // lookup, loop control) then overlaps between the two, and four accumulator sets keep both fed.
    const int ew = warp - EPI_WARP0, quarter = warp & 3, half = ew >> 2;
    const bool affine = p.scale != nullptr || p.shift != nullptr;
    const int pieces = p.c_out >> 4;
    bool bad = false;
    // one 16-column piece: affine, residual, ReLU, convert, store
    auto emit = [&](const uint32_t (&r)[16], int c0, TO* orow, const TO* rrow) {
      float y[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) y[i] = __uint_as_float(r[i]);
      if (affine) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = fmaf(y[i], ctl->sc[c0 + i], ctl->sh[c0 + i]);
      }
      if (rrow) add_residual<TO>(rrow, c0, y, p.c_store, p.vec);
      if (p.relu) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = fmaxf(y[i], 0.f);
      }
      store_piece<TO>(orow, c0, y, p.c_store, p.vec);
    };
    // Destination rows of this thread's row in a unit.  They are requested one unit of this warp
    // ahead: the table comes from DRAM and its latency would otherwise sit between every
    // accumulator set and its stores.
    UnitCursor cur = first;
    if (half) cur.advance(grid, tiles);
    int ab = half % p.nacc, aphase = 0;   // local unit n uses set n % nacc in phase (n / nacc) & 1
    int dnext[MAX_Q];
#pragma unroll
    for (int o = 0; o < MAX_Q; ++o) dnext[o] = -1;
    auto load_dsts = [&](const UnitCursor& c) {
      const int row = c.tile * BLOCK_M + quarter * 32 + lane;
      const int k0 = c.chunk * p.q, qc = min(p.q, p.K - k0);
#pragma unroll
      for (int o = 0; o < MAX_Q; ++o) {
        dnext[o] = -1;
        if (o < qc && row < p.M_in) dnext[o] = p.dst ? __ldg(&p.dst[(int64_t)(k0 + o) * p.M_in + row]) : row;
      }
    };
    if (cur.chunk < p.nchunks) load_dsts(cur);
    while (cur.chunk < p.nchunks) {
      const int qc = min(p.q, p.K - cur.chunk * p.q);
      int dsts[MAX_Q];
#pragma unroll
      for (int o = 0; o < MAX_Q; ++o) dsts[o] = dnext[o];
      UnitCursor nxt = cur;
      nxt.advance(2 * grid, tiles);
      if (nxt.chunk < p.nchunks) load_dsts(nxt);
      if (ok) ok = mbar_wait(bar(&ctl->acc_full[ab]), aphase, p.dev_status);
      if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }  // tcgen05.ld is warp-collective
      tc_fence_after();
      const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * ncols);
#pragma unroll
      for (int o = 0; o < MAX_Q; ++o) {
        if (o >= qc) break;
        int64_t d = dsts[o];
        if (d >= p.num_out) { bad = true; d = -1; }
        TO* orow = reinterpret_cast<TO*>(p.out) + d * p.out_ld;
        const TO* rrow = p.residual ? reinterpret_cast<const TO*>(p.residual) + d * p.res_ld : nullptr;
        for (int g = 0; g < pieces; g += 3) {   // three TMEM loads in flight
          const int c0 = g << 4, c1 = c0 + 16, c2 = c0 + 32;
          const bool has1 = g + 1 < pieces, has2 = g + 2 < pieces;
          uint32_t r0[16], r1[16], r2[16];
          __syncwarp();
          tmem_ld16(trow + (uint32_t)(o * p.c_out + c0), r0);  // executed by every lane of the warp
          if (has1) tmem_ld16(trow + (uint32_t)(o * p.c_out + c1), r1);
          if (has2) tmem_ld16(trow + (uint32_t)(o * p.c_out + c2), r2);
          tmem_ld_wait();
          if (d < 0) continue;
          if (c0 < p.c_store) emit(r0, c0, orow, rrow);
          if (has1 && c1 < p.c_store) emit(r1, c1, orow, rrow);
          if (has2 && c2 < p.c_store) emit(r2, c2, orow, rrow);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(&ctl->acc_empty[ab]));
      ab += 2;
      while (ab >= p.nacc) { ab -= p.nacc; aphase ^= 1; }
      cur = nxt;
    }
    if (bad) wcn_report_bounds(p.dev_status);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, tmem_total);
}

inline int pick_bk(int c_in) { return c_in % 64 == 0 ? 64 : 32; }

// Offsets per chunk, weight buffers, ring depth and accumulator sets for a shape; false when even
// one offset's weights leave no room for the row-tile ring.
bool plan_rows(int K, int c_in, int c_out, RowsParams* p, size_t* smem) {
  const int bk = pick_bk(c_in);
  const int a_bytes = BLOCK_M * bk * 2;
  const int64_t per_offset = (int64_t)c_in * c_out * 2;
  const int fixed = (int)sizeof(RowsControl) + 1024;
  int q = MAX_COLS / c_out < K ? MAX_COLS / c_out : K, nbuf = 0;
  if (q > MAX_Q) q = MAX_Q;
  for (; q >= 1; --q) {
    const int nchunks = (K + q - 1) / q;
    for (int nb = nchunks > 1 ? 2 : 1; nb >= 1 && !nbuf; --nb)
      if (nb * q * per_offset + 4 * a_bytes + fixed <= SMEM_BUDGET) nbuf = nb;
    if (nbuf) break;
  }
  if (!nbuf) return false;
  int64_t stages = (SMEM_BUDGET - fixed - nbuf * q * per_offset) / a_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return false;
  p->q = q; p->nbuf = nbuf; p->stages = (int)stages; p->nchunks = (K + q - 1) / q;
  p->nacc = 512 / (q * c_out) < MAX_ACC ? 512 / (q * c_out) : MAX_ACC;  // q * c_out <= 256: at least two
  *smem = (size_t)(nbuf * q * per_offset + stages * a_bytes + fixed);
  return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    tried = true;
  }
  return fn;
}

template <int BK, bool BF16, typename TO>
int launch_rows(const CUtensorMap& map, const RowsParams& p, size_t smem, unsigned grid, cudaStream_t st) {
  auto kern = conv_rows_tcgen05_kernel<BK, BF16, TO>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET) != cudaSuccess)
      return WCN_ERR_EXECUTION;
    configured[dev] = true;
  }
  kern<<<grid, THREADS, smem, st>>>(map, p);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

}  // namespace

bool wcn_conv_rows_shape_supported(int K, int c_in, int c_out_packed, int dtype, int out_dtype) {
  RowsParams p = {};
  size_t smem = 0;
  return (dtype == WCN_F16 || dtype == WCN_BF16) && (out_dtype == dtype || out_dtype == WCN_F32) && K >= 1 && K <= 32 &&
         c_in >= 32 && c_in % 32 == 0 && c_out_packed >= 16 && c_out_packed <= MAX_COLS && c_out_packed % 16 == 0 &&
         plan_rows(K, c_in, c_out_packed, &p, &smem);
}

int wcn_conv_rows_tcgen05_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed,
                              const int32_t* dst_rows, int64_t num_out, int K, int c_in, int c_out_packed, int c_out,
                              int dtype, const float* scale, const float* shift, const void* residual,
                              int64_t residual_ld, int relu, void* out, int64_t out_ld, int out_dtype,
                              int32_t* dev_status, cudaStream_t st) {
  if (!wcn_conv_rows_shape_supported(K, c_in, c_out_packed, dtype, out_dtype)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (c_out < 1 || c_out > c_out_packed || (!dst_rows && K != 1)) return WCN_ERR_INVALID_PARAMETERS;
  if (!dev_status || !packed || !feats || !out || num_in <= 0 || num_in >= 0x7FFFFFFFll || num_out <= 0)
    return WCN_ERR_INVALID_PARAMETERS;
  // the tensor map wants a 16-byte aligned base and row pitch
  if ((reinterpret_cast<uintptr_t>(feats) & 15) || (feats_ld * 2) % 16 || (reinterpret_cast<uintptr_t>(packed) & 15))
    return WCN_ERR_UNSUPPORTED_CONFIG;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return WCN_ERR_UNSUPPORTED_CONFIG;

  const int64_t osz = out_dtype == WCN_F32 ? 4 : 2;
  auto aligned = [&](int64_t a) {
    return (reinterpret_cast<uintptr_t>(out) % a) == 0 && (out_ld * osz) % a == 0 &&
           (!residual || ((reinterpret_cast<uintptr_t>(residual) % a) == 0 && (residual_ld * osz) % a == 0));
  };
  const int vec = aligned(32) ? 32 : aligned(16) ? 16 : aligned(8) ? 8 : 0;
  RowsParams p = {};
  size_t smem = 0;
  if (!plan_rows(K, c_in, c_out_packed, &p, &smem)) return WCN_ERR_UNSUPPORTED_CONFIG;
  p.vec = vec;
  p.wpacked = (const char*)packed; p.dst = dst_rows; p.M_in = num_in; p.num_out = num_out;
  p.K = K; p.c_in = c_in; p.c_out = c_out_packed; p.c_store = c_out;
  p.tiles = (num_in + BLOCK_M - 1) / BLOCK_M;
  p.units = p.tiles * p.nchunks;
  p.scale = scale; p.shift = shift; p.residual = residual; p.res_ld = residual_ld; p.relu = relu;
  p.out = out; p.out_ld = out_ld; p.dev_status = dev_status;

  const int bk = pick_bk(c_in);
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)c_in, (cuuint64_t)num_in};
  const cuuint64_t strides[1] = {(cuuint64_t)feats_ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)BLOCK_M};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = encode(&map, dtype == WCN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             const_cast<void*>(feats), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return WCN_ERR_UNSUPPORTED_CONFIG;

  const int sms = num_sms();
  const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
  const bool bf = dtype == WCN_BF16;
#define WCN_ROWS_CASE(BKV, BFV, TOV) return launch_rows<BKV, BFV, TOV>(map, p, smem, grid, st)
  if (out_dtype == WCN_F32) {
    if (bk == 64) { if (bf) WCN_ROWS_CASE(64, true, float); else WCN_ROWS_CASE(64, false, float); }
    else          { if (bf) WCN_ROWS_CASE(32, true, float); else WCN_ROWS_CASE(32, false, float); }
  } else if (bf) {
    if (bk == 64) WCN_ROWS_CASE(64, true, __nv_bfloat16); else WCN_ROWS_CASE(32, true, __nv_bfloat16);
  } else {
    if (bk == 64) WCN_ROWS_CASE(64, false, __half); else WCN_ROWS_CASE(32, false, __half);
  }
#undef WCN_ROWS_CASE
}
