// Weight gradient of the sparse convolution on the 5th-generation tensor cores:
//
//     dW[k][ci][co] = sum over output rows m with a neighbour at offset k of
//                     X[nbr[k][m]][ci] * dY[m][co]
//
// i.e. per kernel offset a tall-skinny GEMM X_k^T (C_in x rows) times dY (rows x C_out) whose
// reduction runs over the rows.  Both operands are what the forward kernel already knows how
// to fetch: 128 gathered rows of X and 128 consecutive rows of dY, as swizzled shared-memory
// tiles whose rows are 128-byte (or 64-byte) channel slices.  Read as MN-major operands those
// tiles put the channels on the M / N side of tcgen05.mma and the rows on its K side, so a
// 128-row step is eight K = 16 instructions and nothing is transposed in memory.
//
// The M = 128 side of an instruction holds 128 / CW "units", a unit being the CW = 64 (or 32)
// channel slice of X gathered through ONE offset; consecutive units (offset-major) form a
// group, so a group covers two offsets at C_in = 64, half an offset at C_in = 256, and always
// shares the same dY tile.  A CTA owns (a contiguous range of 128-row steps) x (one group),
// accumulates its [128 x C_out] block in tensor memory and adds it to the fp32 gradient with
// red.global.add (the caller zeroes the gradient; the order of the adds is not fixed, as in
// any split reduction).  Roles: 8 producer warps (cp.async gathers that signal the stage's
// mbarrier when they land), 1 MMA thread, 4 epilogue warps.  Every wait is bounded and
// reports through the device status word.
#include "wcn_common.cuh"
#include "tcgen05_common.cuh"

namespace {

constexpr int WG_ROWS = 128;          // rows per step (K extent of 8 instructions)
constexpr int WG_MAX_STAGES = 4;
constexpr int WG_EPI_WARPS = 4;        // warps 0..3
constexpr int WG_PROD_WARP0 = 4;      // warps 4..11
constexpr int WG_PROD_THREADS = 256;
constexpr int WG_MMA_WARP = 12;
constexpr int WG_THREADS = 416;
static_assert(WG_PROD_WARP0 == WG_EPI_WARPS && WG_THREADS == (WG_MMA_WARP + 1) * 32, "role layout");

struct WgradParams {
  const char* feats;     // [num_in, c_in]
  const char* gout;      // [M, c_out]
  const int32_t* nbr;    // [K][M]
  const int32_t* out_rows;     // slot -> row of gout (tiled table), or null for the identity
  const uint32_t* tile_masks;  // per 128-row step: offsets with any neighbour (null: every step is processed)
  float* gw;             // [K][c_in][c_out] fp32, accumulated into
  int64_t M, num_in;
  int K, c_in, c_out;
  int32_t* dev_status;
  int stages;            // ring depth
  int steps_per_cta;     // 128-row steps per row range
  int cols;              // TMEM columns (power of two >= c_out)
};

struct WgradControl {
  uint64_t full[WG_MAX_STAGES], empty[WG_MAX_STAGES];
  uint64_t acc_full;
  uint32_t tmem_holder;
  int skip;
  int any;  // the accumulator received at least one step
};

template <int RBA, int RBB, bool BF16>
__global__ void __launch_bounds__(WG_THREADS, 1)
conv_wgrad_tcgen05_kernel(const WgradParams p) {
  constexpr int CWA = RBA / 2;              // channels per unit
  constexpr int GU = 128 / CWA;             // units per group (the M = 128 side)
  constexpr int CHA = RBA / 16, CHB = RBB / 16;
  constexpr int A_TILE = WG_ROWS * RBA;     // one unit's tile
  constexpr int B_TILE = WG_ROWS * RBB;     // one dY channel chunk's tile
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int UA = p.c_in / CWA;              // units per offset
  const int NB = p.c_out / (RBB / 2);       // dY channel chunks
  const int total_units = p.K * UA;
  const int unit0 = blockIdx.y * GU;
  const int A_STAGE = GU * A_TILE, B_STAGE = NB * B_TILE;
  const int STAGE = A_STAGE + B_STAGE;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  WgradControl* ctl = reinterpret_cast<WgradControl*>(gen + (size_t)p.stages * STAGE);
  auto bar = [](uint64_t* b) { return smem_u32(b); };

  if (tid == 0) ctl->skip = *(volatile int32_t*)p.dev_status;  // an earlier launch on this status word failed
  __syncthreads();
  if (ctl->skip == (int)WCN_ERR_WAIT_EXPIRED) return;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(bar(&ctl->full[s]), WG_PROD_THREADS); mbar_init(bar(&ctl->empty[s]), 1); }
    mbar_init(bar(&ctl->acc_full), 2);  // the commit of the last MMAs and the issuer's own arrival
    ctl->any = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WG_MMA_WARP) tmem_alloc(smem_u32(&ctl->tmem_holder), (uint32_t)p.cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_holder;

  const int64_t total_steps = (p.M + WG_ROWS - 1) / WG_ROWS;
  const int64_t step0 = (int64_t)blockIdx.x * p.steps_per_cta;
  const int64_t step1 = min(total_steps, step0 + p.steps_per_cta);
  bool ok = true;
  // offsets this group gathers through; a step none of whose rows has a neighbour at any of them
  // contributes nothing and is skipped by every role alike
  uint32_t gmask = 0;
  for (int u = 0; u < GU; ++u)
    if (unit0 + u < total_units) gmask |= 1u << ((unit0 + u) / UA);

  if (warp >= WG_PROD_WARP0 && warp < WG_MMA_WARP) {
    // ================================================================ producers
    const int pt = tid - WG_PROD_WARP0 * 32, pwarp = warp - WG_PROD_WARP0;
    constexpr int RPI = 32 / CHA;                 // tile rows per warp-wide copy instruction
    constexpr int NJ = 16 / RPI;                  // instructions per warp per unit (16 rows per warp)
    const int sub_row = lane / CHA, chunk = lane % CHA;
    uint32_t aoff[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) aoff[j] = tile_offset<RBA>(pwarp * 16 + j * RPI + sub_row, chunk);
    const int PR = p.c_out * 2 / 16;              // 16-byte pieces of a dY row
    const int b_iters = WG_ROWS * PR / WG_PROD_THREADS;
    int slot = 0, phase = 0;
    bool bad = false;
    for (int64_t st = step0; st < step1 && ok; ++st) {
      if (p.tile_masks && !(__ldg(&p.tile_masks[st]) & gmask)) continue;
      const int64_t m0 = st * WG_ROWS;
      // the neighbour indices of this thread's rows, for every unit of the group, before the wait
      int src[GU][NJ];
#pragma unroll
      for (int u = 0; u < GU; ++u) {
        const int unit = unit0 + u;
        const int k = unit / UA;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int64_t m = m0 + pwarp * 16 + j * RPI + sub_row;
          // (the loads of a step are independent and all in flight together: nothing with a side effect sits
          // between them — an index that names no feature row only raises a flag here and is reported once)
          int r = (unit < total_units && m < p.M) ? __ldg(&p.nbr[(int64_t)k * p.M + m]) : -1;
          if (r >= (int)p.num_in) { r = -1; bad = true; }  // counts as absent
          src[u][j] = r;
        }
      }
      if (!mbar_wait_inline(bar(&ctl->empty[slot]), phase ^ 1, p.dev_status)) { ok = false; break; }
      const uint32_t a_dst = base + slot * STAGE;
      const uint32_t b_dst = a_dst + A_STAGE;
#pragma unroll
      for (int u = 0; u < GU; ++u) {
        const int unit = unit0 + u;
        const int slice = unit % UA;
        const char* fbase = p.feats + (int64_t)slice * RBA + chunk * 16;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const bool have = src[u][j] >= 0;
          cp_async16(a_dst + u * A_TILE + aoff[j], have ? fbase + (int64_t)src[u][j] * p.c_in * 2 : p.feats,
                     have ? 16u : 0u);
        }
      }
      for (int i = 0; i < b_iters; ++i) {
        const int q = pt + i * WG_PROD_THREADS;
        const int row = q / PR, piece = q - row * PR;
        const bool have = m0 + row < p.M;
        int64_t grow = m0 + row;
        if (have && p.out_rows) grow = __ldg(&p.out_rows[grow]);
        cp_async16(b_dst + (piece / CHB) * B_TILE + tile_offset<RBB>(row, piece % CHB),
                   have ? p.gout + (grow * p.c_out) * 2 + piece * 16 : p.gout, have ? 16u : 0u);
      }
      cp_async_arrive(bar(&ctl->full[slot]));  // hardware arrives when this thread's copies land
      if (++slot == p.stages) { slot = 0; phase ^= 1; }
    }
    cp_async_drain();
    if (bad) wcn_report_bounds(p.dev_status);
  } else if (warp == WG_MMA_WARP) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      // fp32 accumulate, A and B MN-major (bits 15, 16), N = c_out, M = 128
      const uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) | (1u << 15) | (1u << 16) |
                             ((uint32_t)(p.c_out >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int slot = 0, phase = 0;
      bool any = false;
      for (int64_t st = step0; st < step1 && ok; ++st) {
        if (p.tile_masks && !(__ldg(&p.tile_masks[st]) & gmask)) continue;
        if (!mbar_wait_inline(bar(&ctl->full[slot]), phase, p.dev_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_slot = base + slot * STAGE;
        const uint32_t b_slot = a_slot + A_STAGE;
#pragma unroll
        for (int ks = 0; ks < WG_ROWS / 16; ++ks) {  // 16 rows = two 8-row atoms further down the tiles
          const uint64_t adesc = smem_desc_mn<RBA>(a_slot + ks * 16 * RBA, (uint32_t)A_TILE);
          const uint64_t bdesc = smem_desc_mn<RBB>(b_slot + ks * 16 * RBB, (uint32_t)B_TILE);
          umma_f16(tmem_base, adesc, bdesc, idesc, (any || ks > 0) ? 1u : 0u);
        }
        any = true;
        umma_commit(bar(&ctl->empty[slot]));  // the stage is free once these MMAs have read it
        if (++slot == p.stages) { slot = 0; phase ^= 1; }
      }
      umma_commit(bar(&ctl->acc_full));  // arrives when every MMA above has completed (at once if there were none)
      ctl->any = (any && ok) ? 1 : 0;
      mbar_arrive(bar(&ctl->acc_full));  // publishes `any`
    }
    __syncwarp();
  } else {
    // ================================================================ epilogue (warps 0..3)
    ok = mbar_wait_inline(bar(&ctl->acc_full), 0, p.dev_status);
    if (__all_sync(0xFFFFFFFFu, ok) && ctl->any) {
      tc_fence_after();
      const int row = warp * 32 + lane;            // TMEM lane = position on the M side
      const int unit = unit0 + row / CWA;
      const bool live = unit < total_units;
      const int k = unit / UA, ci = (unit % UA) * CWA + row % CWA;
      float* dst = p.gw + ((int64_t)k * p.c_in + ci) * p.c_out;
      const uint32_t trow = tmem_base + ((uint32_t)(warp * 32) << 16);
      for (int c0 = 0; c0 < p.c_out; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(trow + (uint32_t)c0, r);  // executed by all lanes of the warp
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 16; ++i) atomicAdd(dst + c0 + i, __uint_as_float(r[i]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WG_MMA_WARP) tmem_dealloc(tmem_base, (uint32_t)p.cols);
}

template <int RBA, int RBB, bool BF16>
int launch_wgrad(WgradParams& p, cudaStream_t st) {
  constexpr int CWA = RBA / 2, GU = 128 / CWA;
  const int UA = p.c_in / CWA, NB = p.c_out / (RBB / 2);
  const int groups = (p.K * UA + GU - 1) / GU;
  const size_t stage = (size_t)GU * WG_ROWS * RBA + (size_t)NB * WG_ROWS * RBB;
  const size_t limit = 226 * 1024, fixed = 1024 + sizeof(WgradControl) + 128;
  int stages = (int)((limit - fixed) / stage);
  if (stages > WG_MAX_STAGES) stages = WG_MAX_STAGES;
  if (stages < 2) return WCN_ERR_UNSUPPORTED_CONFIG;
  p.stages = stages;
  int cols = 32;
  while (cols < p.c_out) cols <<= 1;
  p.cols = cols;
  // enough CTAs for a few waves, but at least four steps each so the set-up cost stays small
  const int64_t total_steps = (p.M + WG_ROWS - 1) / WG_ROWS;
  int64_t ranges = (4 * (int64_t)num_sms() + groups - 1) / groups;
  if (ranges > (total_steps + 3) / 4) ranges = (total_steps + 3) / 4;
  if (ranges < 1) ranges = 1;
  p.steps_per_cta = (int)((total_steps + ranges - 1) / ranges);
  ranges = (total_steps + p.steps_per_cta - 1) / p.steps_per_cta;

  auto kern = conv_wgrad_tcgen05_kernel<RBA, RBB, BF16>;
  static bool configured[64] = {};  // per template instance and device: opt in to large shared memory once
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return WCN_ERR_INITIALIZATION;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();
      return WCN_ERR_INITIALIZATION;
    }
    configured[dev] = true;
  }
  dim3 grid((unsigned)ranges, (unsigned)groups);
  kern<<<grid, WG_THREADS, fixed + stages * stage, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

}  // namespace

bool wcn_conv_wgrad_tcgen05_supported(int K, int c_in, int c_out, int dtype) {
  return (dtype == WCN_F16 || dtype == WCN_BF16) && K >= 1 && c_in >= 32 && c_in % 32 == 0 && c_out >= 32 &&
         c_out % 32 == 0 && c_out <= 256 && (int64_t)K * c_in <= 65535ll * 32;
}

int wcn_conv_wgrad_tcgen05(const void* feats, int64_t num_in, const void* grad_out, const int32_t* nbr,
                           const int32_t* out_rows, const uint32_t* tile_masks, int64_t M, int K, int c_in, int c_out, int dtype,
                           float* grad_weight, int32_t* dev_status, cudaStream_t st) {
  if (!wcn_conv_wgrad_tcgen05_supported(K, c_in, c_out, dtype)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (!dev_status || !grad_weight || num_in <= 0 || num_in >= 0x7FFFFFFFll) return WCN_ERR_INVALID_PARAMETERS;
  if ((reinterpret_cast<uintptr_t>(feats) & 15) || (reinterpret_cast<uintptr_t>(grad_out) & 15))
    return WCN_ERR_INVALID_PARAMETERS;
  WgradParams p;
  p.feats = (const char*)feats; p.gout = (const char*)grad_out; p.nbr = nbr; p.out_rows = out_rows; p.tile_masks = K <= 32 ? tile_masks : nullptr; p.gw = grad_weight;
  p.M = M; p.num_in = num_in; p.K = K; p.c_in = c_in; p.c_out = c_out; p.dev_status = dev_status;
  const bool a128 = c_in % 64 == 0, b128 = c_out % 64 == 0, bf = dtype == WCN_BF16;
#define WCN_WG_CASE(A, B, F) if (a128 == (A == 128) && b128 == (B == 128) && bf == F) return launch_wgrad<A, B, F>(p, st);
  WCN_WG_CASE(128, 128, false) WCN_WG_CASE(128, 64, false) WCN_WG_CASE(64, 128, false) WCN_WG_CASE(64, 64, false)
  WCN_WG_CASE(128, 128, true) WCN_WG_CASE(128, 64, true) WCN_WG_CASE(64, 128, true) WCN_WG_CASE(64, 64, true)
#undef WCN_WG_CASE
  return WCN_ERR_UNSUPPORTED_CONFIG;
}
