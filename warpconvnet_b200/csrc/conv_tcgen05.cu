// Output-stationary sparse convolution on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive output rows (the 128 TMEM lanes of an M=128
// tcgen05.mma) and all c_out columns.  It walks the kernel offsets that have at
// least one neighbour among its rows; for each (offset, 64- or 32-channel slice)
// the four producer warps gather the neighbour rows of the feature matrix into a
// K-major, hardware-swizzled shared-memory tile with 16-byte cp.async copies
// (absent neighbours are zero-filled) next to the matching slice of the
// pre-tiled weights, and one thread of a fifth warp issues tcgen05.mma
// instructions that accumulate in fp32 in tensor memory.  When every offset has
// been consumed the producer warps turn into the epilogue: tcgen05.ld the
// accumulator, apply scale/shift (folded BatchNorm or bias), residual add and
// ReLU, convert and store each output row exactly once.  No atomics, no
// split-K workspace, bit-reproducible.
//
// Every wait is bounded: a wait that runs out stores WCN_ERR_WAIT_EXPIRED in the
// device status word, all other waits notice it and the CTA leaves through the
// normal exit path (pending copies drained, tensor memory released).
#include "wcn_common.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int MAX_STAGES = 8;
constexpr int PRODUCERS = 128;        // warps 0..3; also the epilogue warps
constexpr int THREADS = PRODUCERS + 32;
constexpr int MAX_OFFSETS = 27;
constexpr long long kWaitCycles = 4000000000ll;  // about two seconds

struct ConvTcParams {
  const char* feats;
  const char* wpacked;
  const int32_t* nbr;
  int64_t M;
  int K, c_in, c_out;
  const float* scale;
  const float* shift;
  const void* residual;
  int relu;
  void* out;
  int32_t* dev_status;
  uint32_t tmem_cols;
  int block_n;   // output columns per CTA (blockIdx.y selects the column block)
  int stages;    // shared-memory pipeline depth, 2..MAX_STAGES
};

// ------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait.  Returns false when the deadline passed or another thread
// already reported a failure.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t* dev_status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*(volatile int32_t*)dev_status != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      atomicMin(dev_status, (int)WCN_ERR_WAIT_EXPIRED);
      return false;
    }
  }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Arrive on `bar` once all cp.async copies issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory: rows of RB = BK*2 bytes, 8-row atoms of
// 8*RB bytes stacked along M/N, 16-byte chunks XOR-swizzled inside an atom.
//   RB = 128: SWIZZLE_128B (layout code 2), chunk ^= row & 7
//   RB =  64: SWIZZLE_64B  (layout code 4), chunk ^= (row & 7) >> 1
template <int RB> __device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  const int r8 = row & 7;
  const int x = (RB == 128) ? r8 : (r8 >> 1);
  return (uint32_t)((row >> 3) * (8 * RB) + r8 * RB + ((chunk ^ x) << 4));
}
template <int RB> __device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);         // start address, 16-byte units
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)((8 * RB) >> 4) << 32;            // stride byte offset between 8-row atoms
  d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
  d |= (uint64_t)(RB == 128 ? 2 : 4) << 61;        // swizzle mode
  return d;
}

template <typename TO> struct OutVec;
template <> struct OutVec<float> {
  static __device__ __forceinline__ void store(float* p, const float (&y)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
  }
  static __device__ __forceinline__ void load(const float* p, float (&y)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      y[4 * i] = v.x; y[4 * i + 1] = v.y; y[4 * i + 2] = v.z; y[4 * i + 3] = v.w;
    }
  }
};
template <typename T16> struct OutVec16 {
  static __device__ __forceinline__ void store(T16* p, const float (&y)[16]) {
    __align__(16) T16 tmp[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) tmp[i] = wcn_from_float<T16>(y[i]);
    reinterpret_cast<uint4*>(p)[0] = reinterpret_cast<uint4*>(tmp)[0];
    reinterpret_cast<uint4*>(p)[1] = reinterpret_cast<uint4*>(tmp)[1];
  }
  static __device__ __forceinline__ void load(const T16* p, float (&y)[16]) {
    __align__(16) T16 tmp[16];
    reinterpret_cast<uint4*>(tmp)[0] = __ldg(reinterpret_cast<const uint4*>(p));
    reinterpret_cast<uint4*>(tmp)[1] = __ldg(reinterpret_cast<const uint4*>(p) + 1);
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = wcn_to_float<T16>(tmp[i]);
  }
};
template <> struct OutVec<__half> : OutVec16<__half> {};
template <> struct OutVec<__nv_bfloat16> : OutVec16<__nv_bfloat16> {};

// ------------------------------------------------------------------ kernel

template <int BK, bool BF16, typename TO>
__global__ void __launch_bounds__(THREADS, 1) conv_tcgen05_kernel(const ConvTcParams p) {
  constexpr int RB = BK * 2;         // bytes per tile row
  constexpr int CH = RB / 16;        // 16-byte chunks per tile row
  constexpr int RPI = 32 / CH;       // tile rows covered by one warp-wide copy instruction
  constexpr int A_BYTES = BLOCK_M * RB;
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t m0 = (int64_t)blockIdx.x * BLOCK_M;
  const int n0 = blockIdx.y * p.block_n;
  const int BN = p.block_n;
  const int S = p.stages;
  const int KB = p.c_in / BK;
  const int B_BYTES = BN * RB;

  __shared__ int s_skip;  // block-uniform: an earlier launch on this status word failed
  if (tid == 0) s_skip = *(volatile int32_t*)p.dev_status;
  __syncthreads();
  if (s_skip != 0) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_base = base;
  const uint32_t b_base = a_base + S * A_BYTES;
  const uint32_t misc = b_base + S * B_BYTES;
  uint8_t* misc_gen = gen + (misc - base);
  int32_t* rows_idx = reinterpret_cast<int32_t*>(misc_gen);                            // [K][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc_gen + MAX_OFFSETS * BLOCK_M * 4);  // full[S], empty[S], acc
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 1);
  uint32_t* act_mask = holder + 1;
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * MAX_STAGES, acc_bar = full0 + 16 * MAX_STAGES;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, PRODUCERS);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    *act_mask = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(smem_u32(holder), p.tmem_cols);
  __syncthreads();

  // neighbour rows of this tile for every offset, and the set of non-empty offsets
  if (tid < PRODUCERS) {
    const int64_t m = m0 + tid;
    uint32_t mine = 0;
    for (int k = 0; k < p.K; ++k) {
      const int r = m < p.M ? __ldg(&p.nbr[(int64_t)k * p.M + m]) : -1;
      rows_idx[k * BLOCK_M + tid] = r;
      if (__any_sync(0xFFFFFFFFu, r >= 0)) mine |= 1u << k;
    }
    if (lane == 0 && mine) atomicOr(act_mask, mine);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t mask = *act_mask;
  const uint32_t tmem_base = *holder;
  const int T = __popc(mask) * KB;  // pipeline iterations

  bool ok = true;
  if (tid < PRODUCERS) {
    // ---------------- producers: gather A rows + copy the weight slice.
    // A: one warp instruction covers RPI rows x one full tile row each (CH lanes per row),
    //    so every request is a whole RB-byte segment of a feature row.
    const int sub_row = lane / CH, chunk = lane % CH;
    int it = 0;
    uint32_t rest = mask;
    while (rest && ok) {
      const int k = __ffs(rest) - 1;
      rest &= rest - 1;
      const char* asrc[CH];
      uint32_t aoff[CH];
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int row = warp * 32 + j * RPI + sub_row;
        const int src = rows_idx[k * BLOCK_M + row];
        asrc[j] = src >= 0 ? p.feats + (int64_t)src * p.c_in * 2 + chunk * 16 : nullptr;
        aoff[j] = tile_offset<RB>(row, chunk);
      }
      const char* bsrc_k = p.wpacked + ((int64_t)k * KB * p.c_out + n0) * RB;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % S;
        if (!mbar_wait(empty0 + 8 * s, ((it / S) & 1) ^ 1, p.dev_status)) { ok = false; break; }
        const uint32_t a_dst = a_base + s * A_BYTES;
#pragma unroll
        for (int j = 0; j < CH; ++j)
          cp_async16(a_dst + aoff[j], asrc[j] ? asrc[j] + kb * RB : p.feats, asrc[j] ? 16u : 0u);
        const uint32_t b_dst = b_base + s * B_BYTES;
        const char* bsrc = bsrc_k + (int64_t)kb * p.c_out * RB;
        for (int j = tid; j < BN * CH; j += PRODUCERS)
          cp_async16(b_dst + tile_offset<RB>(j / CH, j % CH), bsrc + (int64_t)j * 16, 16u);
        cp_async_arrive(full0 + 8 * s);  // hardware arrives when this thread's copies have landed
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
  } else if (lane == 0) {
    // ---------------- MMA issuer
    const uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BLOCK_M >> 4) << 24);
    for (int it = 0; it < T; ++it) {
      const int s = it % S;
      if (!mbar_wait(full0 + 8 * s, (it / S) & 1, p.dev_status)) { ok = false; break; }
      fence_proxy_async();  // copies were written through the generic proxy, the MMA reads through the async one
      tc_fence_after();
      const uint64_t adesc = smem_desc<RB>(a_base + s * A_BYTES);
      const uint64_t bdesc = smem_desc<RB>(b_base + s * B_BYTES);
#pragma unroll
      for (int kk = 0; kk < BK / 16; ++kk)
        umma_f16(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (it | kk) ? 1u : 0u);
      umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
    }
    if (T > 0 && ok) umma_commit(acc_bar);  // accumulator complete
    else mbar_arrive(acc_bar);
  }

  if (tid < PRODUCERS) {
    // ---------------- epilogue: TMEM -> registers -> global
    if (ok) ok = mbar_wait(acc_bar, 0, p.dev_status);
    tc_fence_after();
    const int64_t m = m0 + tid;
    // tcgen05.ld is warp-collective, so the decision to read must be warp-uniform
    if (__all_sync(0xFFFFFFFFu, ok && *(volatile int32_t*)p.dev_status == 0)) {
      const uint32_t trow = tmem_base + ((uint32_t)(warp * 32) << 16);
      TO* orow = reinterpret_cast<TO*>(p.out) + m * p.c_out + n0;
      const TO* rrow = p.residual ? reinterpret_cast<const TO*>(p.residual) + m * p.c_out + n0 : nullptr;
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float y[16];
        if (T > 0) {
          uint32_t r[16];
          tmem_ld16(trow + (uint32_t)c0, r);  // executed by all lanes of the warp
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) y[i] = __uint_as_float(r[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) y[i] = 0.f;
        }
        if (m < p.M) {
          if (p.scale) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] *= __ldg(&p.scale[n0 + c0 + i]);
          }
          if (p.shift) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] += __ldg(&p.shift[n0 + c0 + i]);
          }
          if (rrow) {
            float res[16];
            OutVec<TO>::load(rrow + c0, res);
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] += res[i];
          }
          if (p.relu) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] = fmaxf(y[i], 0.f);
          }
          OutVec<TO>::store(orow + c0, y);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, p.tmem_cols);
}

// weight[K, c_in, c_out] -> packed[K][c_in/BK][c_out][BK]: every (offset, channel
// slice) becomes one contiguous K-major tile.
template <typename T>
__global__ void pack_weight_kernel(const T* __restrict__ w, T* __restrict__ packed, int K, int c_in, int c_out,
                                   int bk) {
  const int64_t total = (int64_t)K * c_in * c_out;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % bk);
  int64_t r = i / bk;
  const int n = (int)(r % c_out);
  r /= c_out;
  const int kb = (int)(r % (c_in / bk));
  const int k = (int)(r / (c_in / bk));
  packed[i] = w[((int64_t)k * c_in + kb * bk + c) * c_out + n];
}

inline int pick_bk(int c_in) { return c_in % 64 == 0 ? 64 : 32; }

inline size_t smem_bytes(int bk, int block_n, int stages) {
  return 1024 + (size_t)stages * (BLOCK_M + block_n) * bk * 2 + MAX_OFFSETS * BLOCK_M * 4 +
         (2 * MAX_STAGES + 1) * 8 + 64;
}

// Column split: small problems do not have enough 128-row tiles to occupy 148 SMs, so the
// output columns are divided among CTAs (each re-gathers the rows, which stay in L2).
inline int pick_block_n(int64_t tiles, int c_out) {
  int best = c_out;
  for (int split = 1; split <= 8; split *= 2) {
    if (c_out % (16 * split) != 0 || c_out / split < 32) break;
    best = c_out / split;
    if (tiles * split >= 256) break;
  }
  return best;
}

// Pipeline depth: as deep as fits, leaving room for a second CTA per SM when stages are small.
inline int pick_stages(int bk, int block_n) {
  const size_t stage = (size_t)(BLOCK_M + block_n) * bk * 2;
  const size_t budget = stage <= 24 * 1024 ? 96 * 1024 : 204 * 1024;  // <= 96 KiB: two CTAs share an SM
  int s = (int)(budget / stage);
  return s < 2 ? 2 : (s > MAX_STAGES ? MAX_STAGES : s);
}

template <int BK, bool BF16, typename TO>
int launch_tc(ConvTcParams& p, cudaStream_t st) {
  const int64_t tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
  p.block_n = pick_block_n(tiles, p.c_out);
  p.stages = pick_stages(BK, p.block_n);
  uint32_t cols = 32;
  while ((int)cols < p.block_n) cols <<= 1;
  p.tmem_cols = cols;
  const size_t smem = smem_bytes(BK, p.block_n, p.stages);
  auto kern = conv_tcgen05_kernel<BK, BF16, TO>;
  static bool configured[64] = {};  // per template instance and device: opt in to large shared memory once
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return WCN_ERR_INITIALIZATION;
  if (!configured[dev]) {
    // the kernel also has a few bytes of static shared memory, which count against the 227 KiB limit
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();  // do not leave a sticky error for the caller's next CUDA call
      return WCN_ERR_INITIALIZATION;
    }
    configured[dev] = true;
  }
  dim3 grid((unsigned)tiles, (unsigned)(p.c_out / p.block_n));
  kern<<<grid, THREADS, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

}  // namespace

bool wcn_conv_tcgen05_supported(int K, int c_in, int c_out, int dtype, int out_dtype) {
  return (dtype == WCN_F16 || dtype == WCN_BF16) && (out_dtype == dtype || out_dtype == WCN_F32) && K >= 1 &&
         K <= MAX_OFFSETS && c_in >= 32 && c_in % 32 == 0 && c_out >= 16 && c_out <= 256 && c_out % 16 == 0;
}

int64_t wcn_conv_tcgen05_packed_bytes(int K, int c_in, int c_out) { return (int64_t)K * c_in * c_out * 2; }

int wcn_conv_tcgen05_pack(const void* weight, int K, int c_in, int c_out, void* packed, cudaStream_t st) {
  const int64_t total = (int64_t)K * c_in * c_out;
  if (total == 0) return WCN_OK;
  pack_weight_kernel<uint16_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      (const uint16_t*)weight, (uint16_t*)packed, K, c_in, c_out, pick_bk(c_in));
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

int wcn_conv_tcgen05_fwd(const void* feats, const void* packed, const int32_t* nbr, int64_t M, int K, int c_in,
                         int c_out, int dtype, const float* scale, const float* shift, const void* residual,
                         int relu, void* out, int out_dtype, int32_t* dev_status, cudaStream_t st) {
  if (!wcn_conv_tcgen05_supported(K, c_in, c_out, dtype, out_dtype)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (!dev_status || !packed) return WCN_ERR_INVALID_PARAMETERS;
  if ((reinterpret_cast<uintptr_t>(feats) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15))
    return WCN_ERR_INVALID_PARAMETERS;
  ConvTcParams p;
  p.feats = (const char*)feats; p.wpacked = (const char*)packed; p.nbr = nbr;
  p.M = M; p.K = K; p.c_in = c_in; p.c_out = c_out;
  p.scale = scale; p.shift = shift; p.residual = residual; p.relu = relu; p.out = out;
  p.dev_status = dev_status;
  const int bk = pick_bk(c_in);
  const bool bf = dtype == WCN_BF16;
#define WCN_TC_CASE(BKV, BFV, TO) if (bk == BKV && bf == BFV) return launch_tc<BKV, BFV, TO>(p, st);
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
