// Output-stationary sparse convolution on the 5th-generation tensor cores.
//
// A persistent CTA (one per SM) walks "supertiles" of G x 128 consecutive output
// rows.  Each 128-row sub-tile owns one fp32 accumulator in tensor memory (the
// 128 TMEM lanes of an M=128 tcgen05.mma); the accumulators are double-buffered
// when they fit, so the epilogue of one supertile overlaps the main loop of the
// next.  Five warp roles, connected by mbarrier rings:
//  * index warps read the neighbour table of the NEXT supertile (which input row
//    feeds each output row at each kernel offset), stage it in shared memory and
//    derive, per sub-tile, the set of offsets that have any neighbour;
//  * all roles then walk  offsets with a neighbour x channel slices x sub-tiles :
//    one thread fetches the weight slice of (offset, channel slice) ONCE per
//    supertile with a bulk copy (the packed weights hold the swizzled shared-memory
//    image), and eight gather warps copy, for every sub-tile with a neighbour at
//    that offset, the 128 neighbour rows of the feature matrix into a K-major
//    swizzled tile (16-byte cp.async, whole row segments per request, absent rows
//    zero-filled); the copies signal the ring's mbarrier themselves when they land;
//  * one thread issues tcgen05.mma (weight slice shared by the G sub-tiles) and
//    releases ring slots with tcgen05.commit;
//  * epilogue warps read the accumulators with tcgen05.ld, apply scale/shift
//    (folded BatchNorm or bias), residual add and ReLU, convert and store every
//    output row exactly once.  No atomics, bit-reproducible.
//
// Problems with fewer 128-row tiles than multiprocessors divide the kernel offsets of a tile
// among S CTAs ("split-K over kernel offsets": slice s owns the offsets [s*K/S, (s+1)*K/S)).
// Each CTA then leaves its fp32 accumulators in a caller-supplied workspace [S][M][C_out] and a
// second kernel adds the S slices in slice order and runs the epilogue; still no atomics and the
// same bits on every run.
//
// Every wait is bounded: a wait that runs out stores WCN_ERR_WAIT_EXPIRED in the
// device status word, the other waits notice it and the CTA leaves through the
// normal exit path (tensor memory released).
#include "wcn_common.cuh"
#include "tcgen05_common.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int MAX_G = 2;              // sub-tiles per supertile (one per MMA issuer)
constexpr int MAX_RING = 12;          // slots per ring
constexpr int MAX_OFFSETS = 27;
constexpr int EPI_THREADS = 128;      // warps 0..3: TMEM lane quarter = warp index
constexpr int IDX_THREADS = 128;      // warps 4..7: neighbour-table staging
constexpr int GATHER_WARP0 = 8;       // warps 8..15: row gathers
constexpr int GATHER_THREADS = 256;
constexpr int MMA_WARP = 16;          // warps 16, 17: MMA issuers (even / odd sub-tiles); warp 16 owns TMEM
constexpr int MMA_ISSUERS = 2;
constexpr int WEIGHT_WARP = 18;       // weight bulk copies
constexpr int THREADS = 608;

struct ConvTcParams {
  const char* feats;
  bool wide_out, wide_partial, wide_res;   // rows of `out` / the slice workspace / `residual` start on 32-byte boundaries
  const char* wpacked;
  const int32_t* nbr;
  const int32_t* out_rows;  // slot -> output row, or null for the identity
  int64_t M, num_in;
  int64_t in_ld_bytes;      // distance between consecutive feature rows, bytes
  int64_t out_ld, res_ld;   // distance between consecutive output / residual rows, elements
  int K, c_in, c_out;
  const float* scale;
  const float* shift;
  const void* residual;
  int relu;
  void* out;
  int32_t* dev_status;
  int block_n;      // output columns per CTA (blockIdx.y selects the column block)
  int G;            // sub-tiles per supertile: 1, 2 or 4
  int nbuf;         // accumulator sets in TMEM: 1 or 2
  int cols;         // TMEM columns per accumulator (power of two >= block_n)
  int sa, sb;       // ring depths
  int kbc;          // channel slices per ring slot (a slot holds kbc K-major tiles side by side)
  int64_t supertiles;
  int S;            // offset slices per supertile (split-K over kernel offsets); 1 = none
  int64_t units;    // supertiles * S work units, walked by the persistent CTAs
  float* partial;   // [S][M][c_out] fp32 accumulators of the slices (S > 1)
};

// Offsets of slice s of S: bits [s*K/S, (s+1)*K/S).
__device__ __forceinline__ uint32_t slice_mask(int s, int S, int K) {
  if (S <= 1) return 0xFFFFFFFFu;
  const int lo = (s * K) / S, hi = ((s + 1) * K) / S;
  const uint32_t upto_hi = hi >= 32 ? 0xFFFFFFFFu : ((1u << hi) - 1u);
  return upto_hi & ~((1u << lo) - 1u);
}

// 32 bytes in one request: a whole sector per lane.  Every thread of the epilogue writes its own row,
// so a store instruction touches 32 different lines; with 16-byte pieces the L2 gets two half-sector
// writes per sector, with 32-byte ones a single full-sector write.
__device__ __forceinline__ void st_global_32B(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

__device__ __forceinline__ void ld_global_32B(const void* p, uint32_t* v) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(p));
}

// `wide`: the destination is 32-byte aligned (rows start on 32-byte boundaries).
template <typename TO> struct OutVec;
template <> struct OutVec<float> {
  static __device__ __forceinline__ void store(float* p, const float (&y)[16], bool wide) {
    if (wide) {
      st_global_32B(p, reinterpret_cast<const uint32_t*>(y));
      st_global_32B(p + 8, reinterpret_cast<const uint32_t*>(y) + 8);
      return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
  }
  static __device__ __forceinline__ void load(const float* p, float (&y)[16], bool wide) {
    if (wide) {
      ld_global_32B(p, reinterpret_cast<uint32_t*>(y));
      ld_global_32B(p + 8, reinterpret_cast<uint32_t*>(y) + 8);
      return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      y[4 * i] = v.x; y[4 * i + 1] = v.y; y[4 * i + 2] = v.z; y[4 * i + 3] = v.w;
    }
  }
};
template <typename T16> struct OutVec16 {
  static __device__ __forceinline__ void store(T16* p, const float (&y)[16], bool wide) {
    __align__(32) T16 tmp[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) tmp[i] = wcn_from_float<T16>(y[i]);
    if (wide) {
      st_global_32B(p, reinterpret_cast<const uint32_t*>(tmp));
      return;
    }
    reinterpret_cast<uint4*>(p)[0] = reinterpret_cast<uint4*>(tmp)[0];
    reinterpret_cast<uint4*>(p)[1] = reinterpret_cast<uint4*>(tmp)[1];
  }
  static __device__ __forceinline__ void load(const T16* p, float (&y)[16], bool wide) {
    __align__(32) T16 tmp[16];
    if (wide) {
      ld_global_32B(p, reinterpret_cast<uint32_t*>(tmp));
    } else {
      reinterpret_cast<uint4*>(tmp)[0] = __ldg(reinterpret_cast<const uint4*>(p));
      reinterpret_cast<uint4*>(tmp)[1] = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = wcn_to_float<T16>(tmp[i]);
  }
};
template <> struct OutVec<__half> : OutVec16<__half> {};
template <> struct OutVec<__nv_bfloat16> : OutVec16<__nv_bfloat16> {};

// Sub-tiles (bit g) that have a neighbour at offset k, from the per-sub-tile offset masks.
__device__ __forceinline__ uint32_t subtiles_at(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3, int k) {
  return ((m0 >> k) & 1u) | (((m1 >> k) & 1u) << 1) | (((m2 >> k) & 1u) << 2) | (((m3 >> k) & 1u) << 3);
}

// Up to N active offsets taken from the low end of `rest` (bit k = offset k still to do);
// ku[u] = -1 beyond the last one.  Returns how many were taken.
template <int N> __device__ __forceinline__ int pop_offsets(uint32_t& rest, int (&ku)[N]) {
  int n = 0;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    ku[u] = -1;
    if (rest) {
      ku[u] = __ffs(rest) - 1;
      rest &= rest - 1;
      n = u + 1;
    }
  }
  return n;
}

// Ring cursor: slot index and the parity of the phase the slot is in.
struct Ring {
  int slot, phase, depth;
  __device__ __forceinline__ void advance() {
    if (++slot == depth) { slot = 0; phase ^= 1; }
  }
};

// Control block in shared memory.
struct Control {
  uint64_t a_full[MAX_RING], a_empty[MAX_RING];
  uint64_t b_full[MAX_RING], b_empty[MAX_RING];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t info_full[2], info_empty[2];
  uint64_t idx_sync;              // rendezvous of the index threads (bounded, unlike bar.sync)
  uint32_t info_mask[2][MAX_G];   // per staged supertile: non-empty offsets of each sub-tile
  uint32_t mask_acc[2][MAX_G];    // index warps' scratch while building the masks
  uint32_t tmem_holder;
  int skip;
  float sc[256], sh[256];         // this CTA's columns of the epilogue scale / shift (1 / 0 when absent)
};

// ------------------------------------------------------------------ kernel

template <int BK, int KBC, bool SPAN, bool BF16, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
conv_tcgen05_kernel(const ConvTcParams p) {
  constexpr int RB = BK * 2;         // bytes per tile row
  constexpr int CH = RB / 16;        // 16-byte chunks per tile row
  constexpr int RPI = 32 / CH;       // tile rows covered by one warp-wide copy instruction
  constexpr int A_BYTES = BLOCK_M * RB;
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, BN = p.block_n, K = p.K, NBUF = p.nbuf;
  const int n0 = blockIdx.y * BN;
  const int KB = p.c_in / BK;
  const int B_BYTES = BN * RB;         // one weight tile
  constexpr int A_SLOT = KBC * A_BYTES;  // KBC channel slices per ring slot (KBC divides c_in / BK)
  const int B_SLOT = KBC * B_BYTES;
  const int IDX_INTS = G * K * BLOCK_M;  // one staged neighbour table

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_base = base;
  const uint32_t b_base = a_base + p.sa * A_SLOT;
  const uint32_t misc = b_base + p.sb * B_SLOT;
  uint8_t* misc_gen = gen + (misc - base);
  Control* ctl = reinterpret_cast<Control*>(misc_gen);
  int32_t* rows_idx = reinterpret_cast<int32_t*>(misc_gen + sizeof(Control));  // [2][G][K][128]
  auto bar = [](uint64_t* b) { return smem_u32(b); };

  if (tid == 0) ctl->skip = *(volatile int32_t*)p.dev_status;  // an earlier launch on this status word failed
  __syncthreads();
  if (ctl->skip == (int)WCN_ERR_WAIT_EXPIRED) {
    // Nothing is computed after a kernel on this status word gave up.  The rows this CTA would have
    // produced are filled with NaN so that the failure cannot pass for data (with offset slices
    // the second kernel does the same).
    if (p.S == 1) {
      const TO nan = wcn_from_float<TO>(__int_as_float(0x7FC00000));
      for (int64_t st = blockIdx.x; st < p.supertiles; st += gridDim.x) {
        const int64_t m0 = st * G * BLOCK_M;
        const int64_t rows = min((int64_t)G * BLOCK_M, p.M - m0);
        for (int64_t i = tid; i < rows * BN; i += THREADS) {
          const int64_t slot = m0 + i / BN;
          const int64_t m = p.out_rows ? (int64_t)__ldg(&p.out_rows[slot]) : slot;
          reinterpret_cast<TO*>(p.out)[m * p.out_ld + n0 + (int)(i % BN)] = nan;
        }
      }
    }
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < p.sa; ++s) { mbar_init(bar(&ctl->a_full[s]), GATHER_THREADS); mbar_init(bar(&ctl->a_empty[s]), MMA_ISSUERS); }
    for (int s = 0; s < p.sb; ++s) { mbar_init(bar(&ctl->b_full[s]), 1); mbar_init(bar(&ctl->b_empty[s]), MMA_ISSUERS); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(&ctl->acc_full[i]), MMA_ISSUERS);
      mbar_init(bar(&ctl->acc_empty[i]), EPI_THREADS);
      mbar_init(bar(&ctl->info_full[i]), 1);
      mbar_init(bar(&ctl->info_empty[i]), EPI_THREADS + MMA_ISSUERS + 1 + GATHER_THREADS / 32);  // epilogue threads, MMA threads, weight thread, gather warps
    }
    mbar_init(bar(&ctl->idx_sync), IDX_THREADS);
    for (int g = 0; g < MAX_G; ++g) ctl->mask_acc[0][g] = ctl->mask_acc[1][g] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < BN; i += THREADS) {
    ctl->sc[i] = p.scale ? __ldg(&p.scale[n0 + i]) : 1.f;
    ctl->sh[i] = p.shift ? __ldg(&p.shift[n0 + i]) : 0.f;
  }
  const uint32_t tmem_total = (uint32_t)(NBUF * G * p.cols);
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&ctl->tmem_holder), tmem_total < 32 ? 32u : tmem_total);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_holder;

  bool ok = true;
  if (warp >= 4 && warp < GATHER_WARP0) {
    // ================================================================ index warps
    // Stage the neighbour table of a supertile (one supertile ahead of the copies):
    // rows_idx[ib][g][k][row] = input row, or -1 where there is no neighbour.
    // Only the offsets of the unit's slice are read; the others are staged as "no neighbour",
    // so every role downstream sees a supertile that simply has fewer offsets.  An index that
    // does not name a feature row is treated as absent and reported (WCN_ERR_BOUNDS).
    const int itid = tid - EPI_THREADS;
    const int num_in = (int)p.num_in;
    int ib = 0, iphase = 0, sphase = 0;
    bool bad = false;
    for (int64_t wu = blockIdx.x; wu < p.units && ok; wu += gridDim.x) {
      const int64_t st = p.S > 1 ? wu / p.S : wu;
      const uint32_t kmask = slice_mask((int)(wu - st * p.S), p.S, K);
      const int64_t m0 = st * G * BLOCK_M;
      if (!mbar_wait(bar(&ctl->info_empty[ib]), iphase ^ 1, p.dev_status)) { ok = false; break; }
      int32_t* dst = rows_idx + ib * IDX_INTS;
      // The rows of both sub-tiles are requested before either is consumed: a thread's loads are what this
      // role waits for, so twice as many in flight halve the time a table takes.
      const int64_t ma = m0 + itid, mb = m0 + BLOCK_M + itid;
      const bool two = G > 1;
      int ra[MAX_OFFSETS], rb[MAX_OFFSETS];
#pragma unroll
      for (int k = 0; k < MAX_OFFSETS; ++k) {
        const bool want = k < K && ((kmask >> k) & 1u);
        ra[k] = (want && ma < p.M) ? __ldg(&p.nbr[(int64_t)k * p.M + ma]) : -1;
        rb[k] = (want && two && mb < p.M) ? __ldg(&p.nbr[(int64_t)k * p.M + mb]) : -1;
      }
      uint32_t mine_a = 0, mine_b = 0;
#pragma unroll
      for (int k = 0; k < MAX_OFFSETS; ++k) {
        if (k < K) {
          if (ra[k] >= num_in) { ra[k] = -1; bad = true; }
          dst[k * BLOCK_M + itid] = ra[k];
          if (__any_sync(0xFFFFFFFFu, ra[k] >= 0)) mine_a |= 1u << k;
          if (two) {
            if (rb[k] >= num_in) { rb[k] = -1; bad = true; }
            dst[(K + k) * BLOCK_M + itid] = rb[k];
            if (__any_sync(0xFFFFFFFFu, rb[k] >= 0)) mine_b |= 1u << k;
          }
        }
      }
      if (lane == 0 && mine_a) atomicOr(&ctl->mask_acc[ib][0], mine_a);
      if (lane == 0 && mine_b) atomicOr(&ctl->mask_acc[ib][1], mine_b);
      // all index threads meet (bounded: a thread that gave up does not arrive, the others time out)
      mbar_arrive(bar(&ctl->idx_sync));
      if (!mbar_wait(bar(&ctl->idx_sync), sphase, p.dev_status)) { ok = false; break; }
      sphase ^= 1;
      if (itid == 0) {
        for (int g = 0; g < MAX_G; ++g) {
          ctl->info_mask[ib][g] = g < G ? ctl->mask_acc[ib][g] : 0u;
          ctl->mask_acc[ib][g] = 0;  // next use of this entry is two supertiles away, behind info_empty
        }
        mbar_arrive(bar(&ctl->info_full[ib]));  // publishes the table and the masks
      }
      if (++ib == 2) { ib = 0; iphase ^= 1; }
    }
    if (bad) wcn_report_bounds(p.dev_status);
  } else if (warp == WEIGHT_WARP) {
    // ================================================================ weight loader
    if (lane == 0) {
      Ring rb{0, 0, p.sb};
      int ib = 0, iphase = 0;
      for (int64_t wu = blockIdx.x; wu < p.units && ok; wu += gridDim.x) {
        if (!mbar_wait(bar(&ctl->info_full[ib]), iphase, p.dev_status)) { ok = false; break; }
        uint32_t rest = ctl->info_mask[ib][0] | ctl->info_mask[ib][1];
        mbar_arrive(bar(&ctl->info_empty[ib]));  // only the masks were needed
        if (++ib == 2) { ib = 0; iphase ^= 1; }
        // One channel slice per offset (KB == 1) and KBC > 1: a ring slot spans KBC consecutive
        // ACTIVE OFFSETS instead of KBC channel slices of one offset, so narrow layers get the same
        // fat slots as wide ones.  All roles take the offsets off the mask in the same groups.
        while (SPAN && rest && ok) {
          int ku[KBC];
          const int nu = pop_offsets<KBC>(rest, ku);
          if (!mbar_wait(bar(&ctl->b_empty[rb.slot]), rb.phase ^ 1, p.dev_status)) { ok = false; break; }
          const uint32_t fullb = bar(&ctl->b_full[rb.slot]);
          mbar_expect_tx(fullb, (uint32_t)(nu * B_BYTES));
#pragma unroll
          for (int u = 0; u < KBC; ++u)
            if (ku[u] >= 0)
              bulk_copy_g2s(b_base + rb.slot * B_SLOT + u * B_BYTES,
                            p.wpacked + ((int64_t)ku[u] * p.c_out + n0) * RB, (uint32_t)B_BYTES, fullb);
          rb.advance();
        }
        while (!SPAN && rest && ok) {
          const int k = __ffs(rest) - 1;
          rest &= rest - 1;
          const char* bsrc_k = p.wpacked + ((int64_t)k * KB * p.c_out + n0) * RB;
          for (int kb0 = 0; kb0 < KB; kb0 += KBC) {
            // weight tiles (offset k, channel slices kb0..): bulk copies onto one barrier, shared by all sub-tiles
            if (!mbar_wait(bar(&ctl->b_empty[rb.slot]), rb.phase ^ 1, p.dev_status)) { ok = false; break; }
            const uint32_t fullb = bar(&ctl->b_full[rb.slot]);
            mbar_expect_tx(fullb, (uint32_t)(KBC * B_BYTES));
#pragma unroll
            for (int u = 0; u < KBC; ++u)
              bulk_copy_g2s(b_base + rb.slot * B_SLOT + u * B_BYTES, bsrc_k + (int64_t)(kb0 + u) * p.c_out * RB,
                            (uint32_t)B_BYTES, fullb);
            rb.advance();
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= GATHER_WARP0 && warp < MMA_WARP) {
    // ================================================================ gather warps
    const int gwarp = warp - GATHER_WARP0;
    constexpr int ROWS_PER_WARP = BLOCK_M / (GATHER_THREADS / 32);  // 16
    constexpr int NJ = ROWS_PER_WARP / RPI;                          // copy instructions per warp per A slot
    const int sub_row = lane / CH, chunk = lane % CH;
    uint32_t aoff[NJ];  // this thread's fixed (row, chunk) positions inside an A tile
#pragma unroll
    for (int j = 0; j < NJ; ++j) aoff[j] = tile_offset<RB>(gwarp * ROWS_PER_WARP + j * RPI + sub_row, chunk);
    Ring ra{0, 0, p.sa};
    int ib = 0, iphase = 0;
    for (int64_t wu = blockIdx.x; wu < p.units && ok; wu += gridDim.x) {
      if (!mbar_wait(bar(&ctl->info_full[ib]), iphase, p.dev_status)) { ok = false; break; }
      const uint32_t mk0 = ctl->info_mask[ib][0], mk1 = ctl->info_mask[ib][1];
      constexpr uint32_t mk2 = 0u, mk3 = 0u;
      const int32_t* tab = rows_idx + ib * IDX_INTS + gwarp * ROWS_PER_WARP + sub_row;
      uint32_t rest = mk0 | mk1 | mk2 | mk3;
      while (SPAN && rest && ok) {  // slots that span offsets (see the weight loader)
        int ku[KBC];
        pop_offsets<KBC>(rest, ku);
        uint32_t gbu[KBC], gany = 0;
#pragma unroll
        for (int u = 0; u < KBC; ++u) {
          gbu[u] = ku[u] >= 0 ? subtiles_at(mk0, mk1, mk2, mk3, ku[u]) : 0u;
          gany |= gbu[u];
        }
        for (uint32_t gb = gany; gb; gb &= gb - 1) {
          const int g = __ffs(gb) - 1;
          if (!mbar_wait(bar(&ctl->a_empty[ra.slot]), ra.phase ^ 1, p.dev_status)) { ok = false; break; }
          const uint32_t a_dst = a_base + ra.slot * A_SLOT;
          const char* fbase = p.feats + chunk * 16;
#pragma unroll
          for (int u = 0; u < KBC; ++u) {
            if ((gbu[u] >> g) & 1u) {  // sub-tiles of offsets this row block does not have stay unused
              const int32_t* rk = tab + (g * K + ku[u]) * BLOCK_M;
              int src[NJ];
#pragma unroll
              for (int j = 0; j < NJ; ++j) src[j] = rk[j * RPI];
#pragma unroll
              for (int j = 0; j < NJ; ++j) {
                const bool have = src[j] >= 0;
                cp_async16(a_dst + u * A_BYTES + aoff[j], have ? fbase + (int64_t)src[j] * p.in_ld_bytes : p.feats,
                           have ? 16u : 0u);
              }
            }
          }
          cp_async_arrive(bar(&ctl->a_full[ra.slot]));
          ra.advance();
        }
      }
      while (!SPAN && rest && ok) {
        const int k = __ffs(rest) - 1;
        rest &= rest - 1;
        const uint32_t gbits = subtiles_at(mk0, mk1, mk2, mk3, k);
        for (int kb0 = 0; kb0 < KB && ok; kb0 += KBC) {
          for (uint32_t gb = gbits; gb; gb &= gb - 1) {
            const int g = __ffs(gb) - 1;
            if (!mbar_wait(bar(&ctl->a_empty[ra.slot]), ra.phase ^ 1, p.dev_status)) { ok = false; break; }
            const uint32_t a_dst = a_base + ra.slot * A_SLOT;
            const int32_t* rk = tab + (g * K + k) * BLOCK_M;
            int src[NJ];  // all index reads first, so the copies below issue back to back
#pragma unroll
            for (int j = 0; j < NJ; ++j) src[j] = rk[j * RPI];
            const char* fbase = p.feats + (int64_t)kb0 * RB + chunk * 16;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
              const bool have = src[j] >= 0;
              const char* sp = have ? fbase + (int64_t)src[j] * p.in_ld_bytes : p.feats;
#pragma unroll
              for (int u = 0; u < KBC; ++u)  // the row's next channel slices are contiguous in memory
                cp_async16(a_dst + u * A_BYTES + aoff[j], have ? sp + u * RB : sp, have ? 16u : 0u);
            }
            cp_async_arrive(bar(&ctl->a_full[ra.slot]));  // hardware arrives when this thread's copies land
            ra.advance();
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(&ctl->info_empty[ib]));  // this warp is done with the staged table
      if (++ib == 2) { ib = 0; iphase ^= 1; }
    }
    cp_async_drain();
  } else if (warp >= MMA_WARP && warp < MMA_WARP + MMA_ISSUERS) {
    // ================================================================ MMA issuers
    // Two threads share the issue work: issuer w takes the sub-tiles with (g & 1) == w.  Both
    // walk the same slot sequence, both observe and release every row slot and every weight
    // slot, and both sign off the accumulator set.
    const uint32_t issuer = (uint32_t)(warp - MMA_WARP);
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BLOCK_M >> 4) << 24);
      Ring ra{0, 0, p.sa}, rb{0, 0, p.sb};
      int ib = 0, iphase = 0, ab = 0, aphase = 0;
      for (int64_t wu = blockIdx.x; wu < p.units && ok; wu += gridDim.x) {
        if (!mbar_wait(bar(&ctl->info_full[ib]), iphase, p.dev_status)) { ok = false; break; }
        const uint32_t mk0 = ctl->info_mask[ib][0], mk1 = ctl->info_mask[ib][1];
        constexpr uint32_t mk2 = 0u, mk3 = 0u;
        const uint32_t uni = mk0 | mk1 | mk2 | mk3;
        mbar_arrive(bar(&ctl->info_empty[ib]));  // only the masks were needed
        if (++ib == 2) { ib = 0; iphase ^= 1; }
        // the accumulator set must have been read out by the epilogue of its previous use
        if (!mbar_wait(bar(&ctl->acc_empty[ab]), aphase ^ 1, p.dev_status)) { ok = false; break; }
        tc_fence_after();
        uint32_t started = 0;
        uint32_t rest = uni;
        while (SPAN && rest && ok) {  // slots that span offsets (see the weight loader)
          int ku[KBC];
          pop_offsets<KBC>(rest, ku);
          uint32_t gbu[KBC], gany = 0;
#pragma unroll
          for (int u = 0; u < KBC; ++u) {
            gbu[u] = ku[u] >= 0 ? subtiles_at(mk0, mk1, mk2, mk3, ku[u]) : 0u;
            gany |= gbu[u];
          }
          if (!mbar_wait(bar(&ctl->b_full[rb.slot]), rb.phase, p.dev_status)) { ok = false; break; }
          const uint32_t b_slot = b_base + rb.slot * B_SLOT;
          for (uint32_t gb = gany; gb; gb &= gb - 1) {
            const int g = __ffs(gb) - 1;
            if (!mbar_wait(bar(&ctl->a_full[ra.slot]), ra.phase, p.dev_status)) { ok = false; break; }
            if (((uint32_t)g & 1u) != issuer) {  // the other issuer's slot
              mbar_arrive(bar(&ctl->a_empty[ra.slot]));
              ra.advance();
              continue;
            }
            tc_fence_after();
            const uint32_t a_slot = a_base + ra.slot * A_SLOT;
            const uint32_t d = tmem_base + (uint32_t)((ab * G + g) * p.cols);
            uint32_t acc = (started >> g) & 1u;
#pragma unroll
            for (int u = 0; u < KBC; ++u) {
              if ((gbu[u] >> g) & 1u) {
                const uint64_t adesc = smem_desc<RB>(a_slot + u * A_BYTES);
                const uint64_t bdesc = smem_desc<RB>(b_slot + u * B_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)
                  umma_f16(d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                           (acc | (uint32_t)kk) ? 1u : 0u);
                acc = 1u;
              }
            }
            started |= 1u << g;
            umma_commit(bar(&ctl->a_empty[ra.slot]));
            ra.advance();
          }
          umma_commit(bar(&ctl->b_empty[rb.slot]));
          rb.advance();
        }
        while (!SPAN && rest && ok) {
          const int k = __ffs(rest) - 1;
          rest &= rest - 1;
          const uint32_t gbits = subtiles_at(mk0, mk1, mk2, mk3, k);
          for (int kb0 = 0; kb0 < KB && ok; kb0 += KBC) {
            if (!mbar_wait(bar(&ctl->b_full[rb.slot]), rb.phase, p.dev_status)) { ok = false; break; }
            const uint32_t b_slot = b_base + rb.slot * B_SLOT;
            for (uint32_t gb = gbits; gb; gb &= gb - 1) {
              const int g = __ffs(gb) - 1;
              // Both issuers pass every row slot in step: a parity wait is only meaningful for a
              // thread that is never a whole ring lap away from the slot, so the issuer that does
              // not consume a slot still observes its fill and signs it off.
              if (!mbar_wait(bar(&ctl->a_full[ra.slot]), ra.phase, p.dev_status)) { ok = false; break; }
              if (((uint32_t)g & 1u) != issuer) {  // the other issuer's slot
                mbar_arrive(bar(&ctl->a_empty[ra.slot]));
                ra.advance();
                continue;
              }
              tc_fence_after();
              const uint32_t a_slot = a_base + ra.slot * A_SLOT;
              const uint32_t d = tmem_base + (uint32_t)((ab * G + g) * p.cols);
              const uint32_t acc0 = (started >> g) & 1u;
#pragma unroll
              for (int u = 0; u < KBC; ++u) {
                const uint64_t adesc = smem_desc<RB>(a_slot + u * A_BYTES);
                const uint64_t bdesc = smem_desc<RB>(b_slot + u * B_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)
                  umma_f16(d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                           (acc0 | (uint32_t)(u | kk)) ? 1u : 0u);
              }
              started |= 1u << g;
              umma_commit(bar(&ctl->a_empty[ra.slot]));  // slot is free once these MMAs have read it
              ra.advance();
            }
            umma_commit(bar(&ctl->b_empty[rb.slot]));
            rb.advance();
          }
        }
        if (started && ok) umma_commit(bar(&ctl->acc_full[ab]));  // accumulators of this supertile complete
        else mbar_arrive(bar(&ctl->acc_full[ab]));
        if (++ab == NBUF) { ab = 0; aphase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ================================================================ epilogue (warps 0..3)
    int ib = 0, iphase = 0, ab = 0, aphase = 0;
    const bool affine = p.scale != nullptr || p.shift != nullptr;
    // One 16-column piece of this thread's row: affine, residual, ReLU, convert, store.
    auto finish16 = [&](float (&y)[16], int c0, TO* orow, const TO* rrow) {
      if (affine) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 s4 = *reinterpret_cast<const float4*>(&ctl->sc[c0 + 4 * q]);
          const float4 h4 = *reinterpret_cast<const float4*>(&ctl->sh[c0 + 4 * q]);
          y[4 * q + 0] = fmaf(y[4 * q + 0], s4.x, h4.x);
          y[4 * q + 1] = fmaf(y[4 * q + 1], s4.y, h4.y);
          y[4 * q + 2] = fmaf(y[4 * q + 2], s4.z, h4.z);
          y[4 * q + 3] = fmaf(y[4 * q + 3], s4.w, h4.w);
        }
      }
      if (rrow) {
        float res[16];
        OutVec<TO>::load(rrow + c0, res, p.wide_res);
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] += res[i];
      }
      if (p.relu) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = fmaxf(y[i], 0.f);
      }
      OutVec<TO>::store(orow + c0, y, p.wide_out);
    };
    const bool sliced = p.S > 1;  // leave raw fp32 sums for the reduction kernel instead of finishing rows
    // This thread's output rows in the two sub-tiles of a unit.  With rows in tile order they come from
    // `out_rows`, and a load issued when its value is needed costs the epilogue a full memory latency per
    // sub-tile (the gather keeps the memory system busy): the rows of the next unit are read while this one
    // is finished.
    auto unit_rows = [&](int64_t wu, int32_t (&rows)[MAX_G]) {
      const int64_t first = (sliced ? wu / p.S : wu) * G * BLOCK_M + tid;
#pragma unroll
      for (int g = 0; g < MAX_G; ++g) {
        const int64_t slot = first + (int64_t)g * BLOCK_M;
        rows[g] = (g < G && slot < p.M) ? (p.out_rows ? __ldg(&p.out_rows[slot]) : (int32_t)slot) : -1;
      }
    };
    int32_t next_rows[MAX_G];
    if ((int64_t)blockIdx.x < p.units) unit_rows(blockIdx.x, next_rows);
    for (int64_t wu = blockIdx.x; wu < p.units; wu += gridDim.x) {
      const int64_t st = sliced ? wu / p.S : wu;
      int32_t rows[MAX_G];
#pragma unroll
      for (int g = 0; g < MAX_G; ++g) rows[g] = next_rows[g];
      if (wu + gridDim.x < p.units) unit_rows(wu + gridDim.x, next_rows);
      if (ok) ok = mbar_wait(bar(&ctl->info_full[ib]), iphase, p.dev_status);
      const uint32_t gm0 = ok ? ctl->info_mask[ib][0] : 0u, gm1 = ok ? ctl->info_mask[ib][1] : 0u;
      mbar_arrive(bar(&ctl->info_empty[ib]));  // only the masks were needed
      if (++ib == 2) { ib = 0; iphase ^= 1; }
      if (ok) ok = mbar_wait(bar(&ctl->acc_full[ab]), aphase, p.dev_status);
      // tcgen05.ld is warp-collective, so the decision to read must be warp-uniform
      if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
      tc_fence_after();
      const int64_t m0 = st * G * BLOCK_M;
      // (neither loop is unrolled: the epilogue's code is shared by all sub-tiles and column pieces, which
      // keeps the kernel's instruction footprint — five roles run side by side on a multiprocessor — small)
#pragma unroll 1
      for (int g = 0; g < G; ++g) {
        if (m0 + (int64_t)g * BLOCK_M >= p.M) break;
        const uint32_t gmask = g == 0 ? gm0 : gm1;
        const int64_t slot = m0 + (int64_t)g * BLOCK_M + tid;
        const int64_t m = g == 0 ? rows[0] : rows[1];   // -1 past the end: never stored
        const bool live = slot < p.M;
        const uint32_t trow = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)((ab * G + g) * p.cols);
        TO* orow = reinterpret_cast<TO*>(p.out) + m * p.out_ld + n0;
        const TO* rrow = p.residual ? reinterpret_cast<const TO*>(p.residual) + m * p.res_ld + n0 : nullptr;
        // slice wu % S of this row block: [S][M][c_out] fp32, rows in table order (a slice owns all columns)
        float* prow = sliced ? p.partial + (((wu - st * p.S) * p.M + slot) * p.c_out) : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {  // two TMEM loads in flight per wait (BN is a multiple of 16)
          const bool two = c0 + 16 < BN;
          float y0[16], y1[16];
          if (gmask) {
            uint32_t r0[16], r1[16];
            tmem_ld16(trow + (uint32_t)c0, r0);  // executed by all lanes of the warp
            if (two) tmem_ld16(trow + (uint32_t)c0 + 16u, r1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) { y0[i] = __uint_as_float(r0[i]); y1[i] = two ? __uint_as_float(r1[i]) : 0.f; }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) y0[i] = y1[i] = 0.f;
          }
          if (live && sliced) {
            OutVec<float>::store(prow + c0, y0, p.wide_partial);
            if (two) OutVec<float>::store(prow + c0 + 16, y1, p.wide_partial);
          } else if (live) {
            finish16(y0, c0, orow, rrow);
            if (two) finish16(y1, c0 + 16, orow, rrow);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar(&ctl->acc_empty[ab]));   // accumulator set may be overwritten
      if (++ab == NBUF) { ab = 0; aphase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, tmem_total < 32 ? 32u : tmem_total);
}

// weight[K, c_in, c_out] -> packed[K][c_in/BK] tiles of [c_out][BK]: every (offset, channel
// slice) becomes one contiguous K-major tile stored as its swizzled shared-memory image
// (the layout of tile_offset above), so the kernel moves it with a single bulk copy.
template <typename T>
__global__ void pack_weight_kernel(const T* __restrict__ w, T* __restrict__ packed, int K, int c_in, int c_out,
                                   int bk) {
  const int64_t total = (int64_t)K * c_in * c_out;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int n = (int)(i % c_out);
  int64_t r = i / c_out;
  const int cin = (int)(r % c_in);
  const int k = (int)(r / c_in);
  const int kb = cin / bk, c = cin % bk;
  const int rb = bk * 2, chunk = c >> 3, within = c & 7, r8 = n & 7;
  const int x = rb == 128 ? r8 : (r8 >> 1);
  const int64_t tile = ((int64_t)k * (c_in / bk) + kb) * c_out * bk;  // elements
  const int64_t off_bytes = (int64_t)(n >> 3) * (8 * rb) + r8 * rb + ((chunk ^ x) << 4);
  packed[tile + off_bytes / 2 + within] = w[i];
}

// Second pass of a convolution whose kernel offsets were divided among S CTAs per row block:
// adds the S fp32 slices of every output element in slice order (fixed, so the result has the
// same bits on every run) and runs the epilogue.  One thread owns four consecutive columns
// of one table row, so the slices are read and the rows written in full lines.
template <typename TO>
__global__ void conv_slice_reduce_kernel(const float* __restrict__ partial, int S, int64_t M, int c_out,
                                         const int32_t* __restrict__ out_rows, const float* __restrict__ scale,
                                         const float* __restrict__ shift, const TO* __restrict__ residual,
                                         int64_t res_ld, int relu, TO* __restrict__ out, int64_t out_ld,
                                         const int32_t* __restrict__ dev_status) {
  const int quads = c_out >> 2;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M * quads) return;
  const int64_t slot = t / quads;
  const int c = (int)(t - slot * quads) * 4;
  const int64_t m = out_rows ? (int64_t)__ldg(&out_rows[slot]) : slot;
  float y[4];
  if (*dev_status == (int)WCN_ERR_WAIT_EXPIRED) {  // the first pass did not run (or gave up): no data to finish
    y[0] = y[1] = y[2] = y[3] = __int_as_float(0x7FC00000);
  } else {
    const float4* src = reinterpret_cast<const float4*>(partial + slot * c_out + c);
    const int64_t slice = M * (int64_t)c_out / 4;
    float4 acc = __ldcg(src);
    for (int s = 1; s < S; ++s) {
      const float4 v = __ldcg(src + s * slice);
      acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    y[0] = acc.x; y[1] = acc.y; y[2] = acc.z; y[3] = acc.w;
    if (scale || shift) {  // the recipe of the one-pass epilogue: one fused multiply-add
#pragma unroll
      for (int i = 0; i < 4; ++i)
        y[i] = fmaf(y[i], scale ? __ldg(&scale[c + i]) : 1.f, shift ? __ldg(&shift[c + i]) : 0.f);
    }
    if (residual) {
      const TO* r = residual + m * res_ld + c;
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] += wcn_to_float<TO>(r[i]);
    }
    if (relu) {
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] = fmaxf(y[i], 0.f);
    }
  }
  __align__(16) TO o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = wcn_from_float<TO>(y[i]);
  TO* dst = out + m * out_ld + c;
  if (sizeof(TO) == 4) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
  else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
}

inline int pick_bk(int c_in) { return c_in % 64 == 0 ? 64 : 32; }

constexpr int MAX_SLICES = 16;

// Launch geometry.  A problem with fewer 128-row tiles than multiprocessors cannot occupy the
// GPU with one CTA per tile.  With a 3x3x3-sized window there is enough work per tile to divide
// its kernel offsets among S CTAs (split_k: 0 = decide here, 1 = never, >= 2 = that many
// slices); otherwise the output columns are divided among CTAs, each re-gathering the rows,
// which stay in L2 (split_k < 0 forces -split_k column blocks).
bool plan_launch(ConvTcParams& p, int bk, int split_k, size_t* smem, dim3* grid) {
  const int sms = num_sms();
  const int64_t tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
  int S = 1;
  if (split_k >= 2) {
    S = split_k;
  } else if (split_k == 0 && p.K >= 9 && tiles * 2 <= sms) {
    S = (int)(sms / tiles);
    if (S > 8) S = 8;
  }
  if (S > p.K) S = p.K;
  if (S > MAX_SLICES) S = MAX_SLICES;
  int split = 1;
  if (S == 1) {
    if (split_k < 0) {
      split = -split_k;
      if (split > 16 || p.c_out % (16 * split) != 0) return false;
    } else {
      // Column blocks only while they at least double the CTAs that fit: with more than half as many
      // tiles as multiprocessors one full-width CTA per tile is faster (measured: 147 tiles,
      // 128 -> 128 channels, 39 us whole against 59 us in two column blocks).
      while (tiles * split * 2 <= sms && p.c_out % (16 * split * 2) == 0 && p.c_out / (split * 2) >= 32 && split < 8) split *= 2;
    }
  }
  p.S = S;
  p.block_n = p.c_out / split;
  int cols = 32;
  while (cols < p.block_n) cols <<= 1;
  p.cols = cols;
  // Two sub-tiles per supertile (one per issuer).  Four were used for narrow outputs once, to share a weight
  // slice among more rows; narrow layers have tiny weights, and the two extra staged tables (55 KB) are worth
  // more as row slots: 3x3x3 C = 32 / 64 layers measured 11 % faster with two.
  int g = 2;
  while (g > 1 && ((tiles + g - 1) / g) * split * S < 2 * (int64_t)sms) g /= 2;
  const size_t a_unit = (size_t)BLOCK_M * bk * 2, b_unit = (size_t)p.block_n * bk * 2;
  const size_t limit = 226 * 1024;  // the kernels opt in to this much dynamic shared memory
  const int kb_total = p.c_in / bk;
  // Channel slices per ring slot: as many as give a 32 KiB row slot, fewer if the rings would not fit.
  // (with a single slice per offset the slot spans that many active offsets instead)
  int kbc = (int)((32 * 1024) / a_unit);
  if (kb_total > 1 && kbc > kb_total) kbc = kb_total;
  if (kb_total == 1 && kbc > p.K) kbc = p.K;
  if (kbc > 4) kbc = 4;
  if (kbc < 1) kbc = 1;
  while (kb_total > 1 && kb_total % kbc != 0) --kbc;
  size_t fixed = 0, a_stage = 0, b_stage = 0;
  for (;;) {  // two staged neighbour tables + a few row slots and 2 weight slots must fit
    fixed = 1024 + sizeof(Control) + 2 * (size_t)g * p.K * BLOCK_M * 4 + 128;
    a_stage = kbc * a_unit;
    b_stage = kbc * b_unit;
    if (fixed + (kbc > 1 ? 3 : 4) * a_stage + 2 * b_stage <= limit) break;
    if (kbc > 1) {
      do { --kbc; } while (kb_total > 1 && kb_total % kbc != 0);
      continue;
    }
    if (g == 1) return false;
    g /= 2;
  }
  p.kbc = kbc;
  p.G = g;
  p.nbuf = (g * cols * 2 <= 512) ? 2 : 1;
  p.supertiles = (tiles + g - 1) / g;
  p.units = p.supertiles * S;
  const size_t budget = limit - fixed;
  int sb = 3;
  while (sb > 2 && sb * b_stage > budget / 2) --sb;
  int sa = (int)((budget - sb * b_stage) / a_stage);
  if (sa > MAX_RING) sa = MAX_RING;
  if (sa < 2) return false;
  // leftover room goes to the weight ring
  while (sb < 6 && fixed + sa * a_stage + (sb + 1) * b_stage <= limit) ++sb;
  p.sa = sa;
  p.sb = sb;
  *smem = fixed + sa * a_stage + sb * b_stage;
  int64_t gx = p.units;
  const int64_t cap = sms / split > 0 ? sms / split : 1;
  if (gx > cap) gx = cap;
  *grid = dim3((unsigned)gx, (unsigned)split);
  return true;
}

template <int BK, int KBC, bool SPAN, bool BF16, typename TO>
int launch_kbc(const ConvTcParams& p, size_t smem, dim3 grid, cudaStream_t st) {
  auto kern = conv_tcgen05_kernel<BK, KBC, SPAN, BF16, TO>;
  static bool configured[64] = {};  // per template instance and device: opt in to large shared memory once
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return WCN_ERR_INITIALIZATION;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();  // do not leave a sticky error for the caller's next CUDA call
      return WCN_ERR_INITIALIZATION;
    }
    configured[dev] = true;
  }
  kern<<<grid, THREADS, smem, st>>>(p);
  if (cudaGetLastError() != cudaSuccess) return WCN_ERR_EXECUTION;
  if (p.S > 1) {
    const int64_t threads = p.M * (p.c_out >> 2);
    conv_slice_reduce_kernel<TO><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(
        p.partial, p.S, p.M, p.c_out, p.out_rows, p.scale, p.shift, reinterpret_cast<const TO*>(p.residual), p.res_ld,
        p.relu, reinterpret_cast<TO*>(p.out), p.out_ld, p.dev_status);
    if (cudaGetLastError() != cudaSuccess) return WCN_ERR_EXECUTION;
  }
  return WCN_OK;
}

template <int BK, bool BF16, typename TO>
int launch_tc(ConvTcParams& p, int split_k, void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  size_t smem = 0;
  dim3 grid;
  if (!plan_launch(p, BK, split_k, &smem, &grid)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (p.S > 1) {
    const int64_t need = (int64_t)p.S * p.M * p.c_out * (int64_t)sizeof(float);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
      return WCN_ERR_INVALID_PARAMETERS;
    p.partial = reinterpret_cast<float*>(workspace);
  }
  // SPAN: the whole C_in is one slice and a ring slot holds KBC consecutive active offsets; otherwise a
  // slot holds KBC channel slices of one offset.  A compile-time choice, so that every role's loop
  // carries only the form it runs.
  if (p.kbc > 1 && p.c_in == BK) {
    switch (p.kbc) {
      case 2: return launch_kbc<BK, 2, true, BF16, TO>(p, smem, grid, st);
      case 3: return launch_kbc<BK, 3, true, BF16, TO>(p, smem, grid, st);
      case 4: return launch_kbc<BK, 4, true, BF16, TO>(p, smem, grid, st);
      default: return WCN_ERR_UNSUPPORTED_CONFIG;
    }
  }
  switch (p.kbc) {
    case 1: return launch_kbc<BK, 1, false, BF16, TO>(p, smem, grid, st);
    case 2: return launch_kbc<BK, 2, false, BF16, TO>(p, smem, grid, st);
    case 3: return launch_kbc<BK, 3, false, BF16, TO>(p, smem, grid, st);
    case 4: return launch_kbc<BK, 4, false, BF16, TO>(p, smem, grid, st);
    default: return WCN_ERR_UNSUPPORTED_CONFIG;
  }
}

// A barrier phase that cannot complete (one arrival of two), waited for with a short limit:
// the wait has to give up, report WCN_ERR_WAIT_EXPIRED and let the kernel end normally.
__global__ void bounded_wait_probe_kernel(long long limit_cycles, int32_t* dev_status, int32_t* gave_up) {
  __shared__ uint64_t probe_bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&probe_bar), 2);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_arrive(smem_u32(&probe_bar));
  if (threadIdx.x == 32) {
    const bool done = mbar_wait_limit(smem_u32(&probe_bar), 0, dev_status, limit_cycles);
    if (gave_up) *gave_up = done ? 0 : 1;
  }
}

}  // namespace

extern "C" int wcn_selftest_bounded_wait(int64_t limit_cycles, int32_t* dev_status, int32_t* gave_up, void* stream) {
  if (!dev_status || limit_cycles < 1000 || limit_cycles > 2000000000ll) return WCN_ERR_INVALID_PARAMETERS;
  bounded_wait_probe_kernel<<<1, 64, 0, wcn_stream(stream)>>>((long long)limit_cycles, dev_status, gave_up);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

bool wcn_conv_tcgen05_supported(int K, int c_in, int c_out, int dtype, int out_dtype) {
  return (dtype == WCN_F16 || dtype == WCN_BF16) && (out_dtype == dtype || out_dtype == WCN_F32) && K >= 1 &&
         K <= MAX_OFFSETS && c_in >= 32 && c_in % 32 == 0 && c_out >= 16 && c_out <= 256 && c_out % 16 == 0;
}

int64_t wcn_conv_tcgen05_packed_bytes(int K, int c_in, int c_out) { return (int64_t)K * c_in * c_out * 2; }

// Bytes of slice workspace wcn_conv_tcgen05_fwd needs for this problem (0: one pass).
int64_t wcn_conv_tcgen05_workspace_bytes(int64_t M, int K, int c_in, int c_out, int split_k) {
  ConvTcParams p = {};
  p.M = M; p.K = K; p.c_in = c_in; p.c_out = c_out;
  size_t smem = 0;
  dim3 grid;
  if (M <= 0 || !plan_launch(p, pick_bk(c_in), split_k, &smem, &grid) || p.S <= 1) return 0;
  return (int64_t)p.S * M * c_out * (int64_t)sizeof(float);
}

int wcn_conv_tcgen05_pack(const void* weight, int K, int c_in, int c_out, void* packed, cudaStream_t st) {
  const int64_t total = (int64_t)K * c_in * c_out;
  if (total == 0) return WCN_OK;
  pack_weight_kernel<uint16_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      (const uint16_t*)weight, (uint16_t*)packed, K, c_in, c_out, pick_bk(c_in));
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

int wcn_conv_tcgen05_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed, const int32_t* nbr,
                         const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype,
                         const float* scale, const float* shift, const void* residual, int64_t residual_ld, int relu,
                         void* out, int64_t out_ld, int out_dtype, int split_k, void* workspace,
                         int64_t workspace_bytes, int32_t* dev_status, cudaStream_t st) {
  if (!wcn_conv_tcgen05_supported(K, c_in, c_out, dtype, out_dtype)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (!dev_status || !packed || num_in <= 0 || num_in >= 0x7FFFFFFFll || M >= 0x7FFFFFFFll) return WCN_ERR_INVALID_PARAMETERS;
  const int64_t osz = out_dtype == WCN_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(feats) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15) ||
      feats_ld < c_in || (feats_ld * 2) % 16 || out_ld < c_out || (out_ld * osz) % 16 ||
      (residual && (residual_ld < c_out || (residual_ld * osz) % 16)))
    return WCN_ERR_INVALID_PARAMETERS;
  ConvTcParams p = {};
  p.feats = (const char*)feats; p.wpacked = (const char*)packed; p.nbr = nbr; p.out_rows = out_rows;
  p.M = M; p.num_in = num_in; p.K = K; p.c_in = c_in; p.c_out = c_out;
  p.in_ld_bytes = feats_ld * 2; p.out_ld = out_ld; p.res_ld = residual_ld;
  p.scale = scale; p.shift = shift; p.residual = residual; p.relu = relu; p.out = out;
  p.dev_status = dev_status;
  p.wide_out = (reinterpret_cast<uintptr_t>(out) & 31) == 0 && (out_ld * osz) % 32 == 0;
  p.wide_res = residual && (reinterpret_cast<uintptr_t>(residual) & 31) == 0 && (residual_ld * osz) % 32 == 0;
  p.wide_partial = (reinterpret_cast<uintptr_t>(workspace) & 31) == 0;   // its rows are c_out fp32 values: 64-byte multiples
  const int bk = pick_bk(c_in);
  const bool bf = dtype == WCN_BF16;
#define WCN_TC_CASE(BKV, BFV, TO) \
  if (bk == BKV && bf == BFV) return launch_tc<BKV, BFV, TO>(p, split_k, workspace, workspace_bytes, st);
  if (out_dtype == WCN_F32) {
    WCN_TC_CASE(64, false, float) WCN_TC_CASE(64, true, float) WCN_TC_CASE(32, false, float) WCN_TC_CASE(32, true, float)
  } else if (bf) {
    WCN_TC_CASE(64, true, __nv_bfloat16) WCN_TC_CASE(32, true, __nv_bfloat16)
  } else {
    WCN_TC_CASE(64, false, __half) WCN_TC_CASE(32, false, __half)
  }
#undef WCN_TC_CASE
  return WCN_ERR_UNSUPPORTED_CONFIG;
}
