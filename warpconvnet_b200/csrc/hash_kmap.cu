// Coordinate hash table, distinct/strided coordinates, kernel-map generation and
// Morton code.  All of it is integer, bandwidth-bound work: one 16-byte key per
// slot so a probe is one 32-byte sector, coalesced int4 query loads, warp-ballot
// compaction, no host synchronisation inside the library.
#include <atomic>

#include "wcn_common.cuh"

namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------ 128-bit CAS

__device__ __forceinline__ int4 cas128(int4* addr, int4 cmp, int4 val) {
  unsigned long long clo = ((unsigned long long)(uint32_t)cmp.y << 32) | (uint32_t)cmp.x;
  unsigned long long chi = ((unsigned long long)(uint32_t)cmp.w << 32) | (uint32_t)cmp.z;
  unsigned long long vlo = ((unsigned long long)(uint32_t)val.y << 32) | (uint32_t)val.x;
  unsigned long long vhi = ((unsigned long long)(uint32_t)val.w << 32) | (uint32_t)val.z;
  unsigned long long olo, ohi;
  asm volatile(
      "{\n\t"
      ".reg .b128 c, v, o;\n\t"
      "mov.b128 c, {%2, %3};\n\t"
      "mov.b128 v, {%4, %5};\n\t"
      "atom.global.relaxed.gpu.cas.b128 o, [%6], c, v;\n\t"
      "mov.b128 {%0, %1}, o;\n\t"
      "}"
      : "=l"(olo), "=l"(ohi)
      : "l"(clo), "l"(chi), "l"(vlo), "l"(vhi), "l"(addr)
      : "memory");
  int4 old;
  old.x = (int)(uint32_t)olo;
  old.y = (int)(uint32_t)(olo >> 32);
  old.z = (int)(uint32_t)ohi;
  old.w = (int)(uint32_t)(ohi >> 32);
  return old;
}

__device__ __forceinline__ int4 load_key(const int32_t* __restrict__ keys, int64_t i, int sx, int sy,
                                         int sz) {
  int4 k = __ldg(reinterpret_cast<const int4*>(keys) + i);
  if (sx != 1) k.y = wcn_floordiv(k.y, sx);
  if (sy != 1) k.z = wcn_floordiv(k.z, sy);
  if (sz != 1) k.w = wcn_floordiv(k.w, sz);
  return k;
}

// ------------------------------------------------------------------ table build / search

// The table buffer ends with one flag word behind the values: tvals[cap] != 0 when a key was
// inserted more than once.
__global__ void hash_clear_kernel(int4* tkeys, int* tvals, int64_t cap, const int32_t* __restrict__ skip_if) {
  if (skip_if && __ldg(skip_if) != 0) return;  // the caller's brick table is usable: this table will not be probed
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cap) {
    tkeys[i] = make_int4(WCN_EMPTY_BATCH, 0, 0, 0);
    tvals[i] = INT_MAX;
  }
  if (i == 0) tvals[cap] = 0;
}

template <int METHOD>
__global__ void hash_insert_kernel(const int32_t* __restrict__ keys, int64_t n, int sx, int sy, int sz,
                                   int4* tkeys, int* tvals, uint32_t cap, int32_t* dev_status,
                                   const int32_t* __restrict__ skip_if) {
  if (skip_if && __ldg(skip_if) != 0) return;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 key = load_key(keys, i, sx, sy, sz);
  const int4 empty = make_int4(WCN_EMPTY_BATCH, 0, 0, 0);
  uint32_t slot = wcn_slot(wcn_hash4<METHOD>(key), cap);
  for (uint32_t p = 0; p < cap; ++p) {
    // A plain 16-byte load may race with another thread's 128-bit CAS on the same slot.  It relies
    // on an aligned 16-byte global load being single-copy atomic (it is one memory transaction on
    // this architecture), so it sees either the empty marker or a whole key, never a mix; and a
    // stale "empty" is harmless because the CAS below re-reads the slot and returns what is there.
    int4 cur = __ldcg(&tkeys[slot]);
    bool claimed = false;
    if (cur.x == WCN_EMPTY_BATCH) {
      cur = cas128(&tkeys[slot], empty, key);
      claimed = cur.x == WCN_EMPTY_BATCH;
    }
    if (claimed || wcn_key_eq(cur, key)) {
      atomicMin(&tvals[slot], (int)i);  // smallest row index wins: deterministic
      if (!claimed) tvals[cap] = 1;     // the key was there already: the keys are not distinct
      return;
    }
    slot = (slot + 1 == cap) ? 0u : slot + 1;
  }
  if (dev_status) atomicMin(dev_status, (int)WCN_ERR_HASH_OVERFLOW);
}

template <int METHOD>
__global__ void hash_search_kernel(const int4* __restrict__ tkeys, const int* __restrict__ tvals,
                                   uint32_t cap, const int32_t* __restrict__ queries, int64_t nq,
                                   int32_t* __restrict__ results) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq) return;
  const int4 q = __ldg(reinterpret_cast<const int4*>(queries) + i);
  results[i] = wcn_lookup<METHOD>(tkeys, tvals, cap, q);
}

// ------------------------------------------------------------------ block scan helpers

// Exclusive prefix of `v` over the block (blockDim.x <= 1024, multiple of 32);
// the block total is returned through `total` (valid in every thread).
__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  __shared__ int warp_sums[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < nwarps ? warp_sums[lane] : 0;
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xFFFFFFFFu, wi, d);
      if (lane >= d) wi += t;
    }
    warp_sums[lane] = wi - w;  // exclusive prefix of warp sums
  }
  __syncthreads();
  int result = incl - v + warp_sums[warp];
  __shared__ int block_total;  // = exclusive prefix of the last thread + its value
  if (threadIdx.x == blockDim.x - 1) block_total = result + v;
  __syncthreads();
  *total = block_total;
  return result;
}

// In-place exclusive scan of each row of data[rows, len]; totals[row] = row sum.
__global__ void scan_rows_kernel(int* data, int64_t len, int* totals) {
  int* row = data + (int64_t)blockIdx.x * len;
  int carry = 0;
  for (int64_t base = 0; base < len; base += blockDim.x) {
    int64_t i = base + threadIdx.x;
    int v = i < len ? row[i] : 0;
    int total;
    int ex = block_exclusive_scan(v, &total);
    if (i < len) row[i] = carry + ex;
    carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

__global__ void offsets_from_totals_kernel(const int* totals, int rows, int32_t* offsets) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int acc = 0;
    offsets[0] = 0;
    for (int k = 0; k < rows; ++k) {
      acc += totals[k];
      offsets[k + 1] = acc;
    }
  }
}

// ------------------------------------------------------------------ distinct rows

struct UniqueWs {
  int* rep;           // [n] row index of the first occurrence of each row's key
  int* rank_of;       // [n] output position of a first-occurrence row
  int* block_counts;  // [nblk] then scanned in place
  int* total;         // [1]
  int64_t nblk;
};

__host__ __device__ inline int64_t unique_nblk(int64_t n) { return (n + kThreads - 1) / kThreads; }

inline UniqueWs unique_ws(void* ws, int64_t n) {
  UniqueWs w;
  w.nblk = unique_nblk(n);
  w.rep = reinterpret_cast<int*>(ws);
  w.rank_of = w.rep + n;
  w.block_counts = w.rank_of + n;
  w.total = w.block_counts + w.nblk;
  return w;
}

template <int METHOD>
__global__ void unique_mark_kernel(const int32_t* __restrict__ coords, int64_t n, int sx, int sy, int sz,
                                   const int4* __restrict__ tkeys, const int* __restrict__ tvals,
                                   uint32_t cap, int* __restrict__ rep, int* __restrict__ block_counts) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int first = 0;
  if (i < n) {
    const int4 key = load_key(coords, i, sx, sy, sz);
    const int r = wcn_lookup<METHOD>(tkeys, tvals, cap, key);
    rep[i] = r;
    first = (r == (int)i);
  }
  int c = __syncthreads_count(first);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = c;
}

__global__ void store_total_kernel(const int* total, int64_t* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *out = (int64_t)(*total);
}

__global__ void unique_emit_kernel(const int32_t* __restrict__ coords, int64_t n, int sx, int sy, int sz,
                                   const int* __restrict__ rep, const int* __restrict__ block_prefix,
                                   int* __restrict__ rank_of, int32_t* __restrict__ out_coords,
                                   int32_t* __restrict__ unique_index) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool first = (i < n) && (rep[i] == (int)i);
  int total;
  const int ex = block_exclusive_scan(first ? 1 : 0, &total);
  if (first) {
    const int pos = block_prefix[blockIdx.x] + ex;
    rank_of[i] = pos;
    reinterpret_cast<int4*>(out_coords)[pos] = load_key(coords, i, sx, sy, sz);
    if (unique_index) unique_index[pos] = (int)i;
  }
}

__global__ void unique_parent_kernel(int64_t n, const int* __restrict__ rep, const int* __restrict__ rank_of,
                                     int32_t* __restrict__ parent) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int r = rep[i];
    parent[i] = r >= 0 ? rank_of[r] : -1;
  }
}

// ------------------------------------------------------------------ kernel map

struct KernelGeom {
  int sx, sy, sz;  // multiply output coordinates by this
  int kx, ky, kz;
  int cx, cy, cz;  // centre: size/2 for odd sizes, 0 for even
  int dx, dy, dz;  // dilation: spacing of the window positions
};

// One thread per (query m, offset k); m runs along the warp so the query load
// and the nbr store are coalesced.  grid = (ceil(M/256), K).  COUNT: also leave the number
// of hits of every block for the compaction.
template <int METHOD, bool COUNT>
__global__ void kmap_search_kernel(const int4* __restrict__ tkeys, const int* __restrict__ tvals,
                                   uint32_t cap, const int32_t* __restrict__ queries, int64_t M,
                                   KernelGeom g, int32_t* __restrict__ nbr,
                                   int* __restrict__ block_counts) {
  const int k = blockIdx.y;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int found = -1;
  if (m < M) {
    int4 q = __ldg(reinterpret_cast<const int4*>(queries) + m);
    const int l = k % g.kz, j = (k / g.kz) % g.ky, i = k / (g.kz * g.ky);
    q.y = q.y * g.sx + (i - g.cx) * g.dx;
    q.z = q.z * g.sy + (j - g.cy) * g.dy;
    q.w = q.w * g.sz + (l - g.cz) * g.dz;
    found = wcn_lookup<METHOD>(tkeys, tvals, cap, q);
    nbr[(int64_t)k * M + m] = found;
  }
  if (COUNT) {
    const int c = __syncthreads_count(found >= 0);
    if (threadIdx.x == 0) block_counts[(int64_t)k * gridDim.x + blockIdx.x] = c;
  }
}

// Map of a coordinate set onto itself (the queries are the table's own keys, in row order;
// stride 1, odd window).  When the keys are distinct the map is symmetric: row m sees row i at
// offset k exactly when row i sees row m at the mirrored offset K-1-k.  Only the first half of
// the offsets and the centre are probed; a hit also fills the mirrored entry, whose rows were
// set to -1 beforehand.  With repeated keys (flag behind the table values) every offset is
// probed as in kmap_search_kernel.
template <int METHOD>
__global__ void kmap_search_self_kernel(const int4* __restrict__ tkeys, const int* __restrict__ tvals,
                                        uint32_t cap, const int32_t* __restrict__ queries, int64_t M,
                                        KernelGeom g, int K, int32_t* __restrict__ nbr) {
  const int k = blockIdx.y;
  const bool distinct = __ldg(&tvals[cap]) == 0;
  if (distinct && k > K / 2) return;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  int4 q = __ldg(reinterpret_cast<const int4*>(queries) + m);
  const int l = k % g.kz, j = (k / g.kz) % g.ky, i = k / (g.kz * g.ky);
  q.y += (i - g.cx) * g.dx;
  q.z += (j - g.cy) * g.dy;
  q.w += (l - g.cz) * g.dz;
  const int found = wcn_lookup<METHOD>(tkeys, tvals, cap, q);
  nbr[(int64_t)k * M + m] = found;
  if (distinct && k < K / 2 && found >= 0) nbr[(int64_t)(K - 1 - k) * M + found] = (int32_t)m;
}

// Per-block hit counts of a dense neighbour table, in the layout kmap_search_kernel<.., true> leaves.
__global__ void kmap_count_kernel(const int32_t* __restrict__ nbr, int64_t M, int* __restrict__ block_counts) {
  const int k = blockIdx.y;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int c = __syncthreads_count(m < M && __ldg(&nbr[(int64_t)k * M + m]) >= 0);
  if (threadIdx.x == 0) block_counts[(int64_t)k * gridDim.x + blockIdx.x] = c;
}

__global__ void kmap_compact_kernel(const int32_t* __restrict__ nbr, int64_t M,
                                    const int* __restrict__ block_prefix,
                                    const int32_t* __restrict__ offsets, int32_t* __restrict__ in_maps,
                                    int32_t* __restrict__ out_maps) {
  const int k = blockIdx.y;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int v = m < M ? __ldg(&nbr[(int64_t)k * M + m]) : -1;
  int total;
  const int ex = block_exclusive_scan(v >= 0 ? 1 : 0, &total);
  if (v >= 0) {
    const int64_t pos = (int64_t)offsets[k] + block_prefix[(int64_t)k * gridDim.x + blockIdx.x] + ex;
    in_maps[pos] = v;
    out_maps[pos] = (int32_t)m;
  }
}

__global__ void nbr_from_maps_kernel(const int32_t* __restrict__ in_maps,
                                     const int32_t* __restrict__ out_maps,
                                     const int32_t* __restrict__ offsets, int K, int64_t L, int64_t M,
                                     int32_t* __restrict__ nbr) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= L) return;
  int lo = 0, hi = K;  // largest k with offsets[k] <= p
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if ((int64_t)__ldg(&offsets[mid]) <= p) lo = mid; else hi = mid;
  }
  const int32_t o = out_maps[p];
  if (o >= 0 && o < M) nbr[(int64_t)lo * M + o] = in_maps[p];
}

__global__ void nbr_transpose_kernel(const int32_t* __restrict__ nbr_fwd, int64_t M, int64_t N,
                                     int32_t* __restrict__ nbr_t) {
  const int k = blockIdx.y;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const int v = __ldg(&nbr_fwd[(int64_t)k * M + m]);
  if (v >= 0 && v < N) nbr_t[(int64_t)k * N + v] = (int32_t)m;
}

// ------------------------------------------------------------------ tile order

// Rows of one window of consecutive output rows are reordered by their neighbour-presence mask
// (bit k = offset k has a neighbour), ties by row.  Rows with the same set of present offsets
// become adjacent, so a 128-row tile of the reordered table has far fewer offsets with any
// neighbour than a tile of consecutive rows, and the convolution skips a (tile, offset) pair
// that has none.  The window bounds how far a row moves, which keeps the gather footprint of a
// tile local.  Windows of 16384 rows (tables of more than 4096 rows) leave 7-9 % fewer (tile,
// offset) pairs than windows of 4096 on room scans (11.1 / 13.0 / 16.5 offsets per tile at 2, 4 and
// 8 cm against 11.9 / 14.1 / 18.2).
constexpr int kTileWindowSmall = 4096, kTileWindowLarge = 16384;
constexpr int kTileOrderThreads = 1024;
constexpr int kTileCopyOffsets = 3;  // offsets per block of the permuted copy

// Pass 1: presence mask of every output row (one thread per row, all loads in flight).
__global__ void kmap_row_mask_kernel(const int32_t* __restrict__ nbr, int64_t M, int K, uint32_t* __restrict__ masks) {
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  int v[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) v[k] = k < K ? __ldg(&nbr[(int64_t)k * M + m]) : -1;
  uint32_t mask = 0;
  if (K == 27) {
    // Sort key of a 3x3x3 window: the centre in bit 0, then the 6 face, 12 edge and 8 corner offsets, so that
    // the rarest offsets are the most significant bits and rows that share them end up in the same tiles
    // (2-4 % fewer (tile, offset) pairs than offsets in index order).  Only the order of the rows depends on it.
#pragma unroll
    for (int k = 0; k < 27; ++k) {
      const int ax = (k / 9 != 1) + ((k / 3) % 3 != 1) + (k % 3 != 1);   // 0 centre, 1 face, 2 edge, 3 corner
      int pos = 0;   // offsets of a lower class, and earlier ones of the same class, come first
#pragma unroll
      for (int q = 0; q < 27; ++q) {
        const int aq = (q / 9 != 1) + ((q / 3) % 3 != 1) + (q % 3 != 1);
        pos += (aq < ax) || (aq == ax && q < k);
      }
      mask |= (uint32_t)(v[k] >= 0) << pos;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 32; ++k) mask |= (uint32_t)(v[k] >= 0) << k;
  }
  masks[m] = mask;
}

// Offsets with any neighbour among 128 consecutive rows of the table (one block per 128 rows):
// what a kernel that walks the table in 128-row steps may skip.
__global__ void kmap_tile_mask_kernel(const int32_t* __restrict__ nbr, int64_t M, int K, uint32_t* __restrict__ masks) {
  __shared__ uint32_t part[4];
  const int64_t m = (int64_t)blockIdx.x * 128 + threadIdx.x;
  uint32_t mask = 0;
  if (m < M) {
    int v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = k < K ? __ldg(&nbr[(int64_t)k * M + m]) : -1;
#pragma unroll
    for (int k = 0; k < 32; ++k) mask |= (uint32_t)(v[k] >= 0) << k;
  }
  mask = __reduce_or_sync(0xFFFFFFFFu, mask);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = mask;
  __syncthreads();
  if (threadIdx.x == 0) masks[blockIdx.x] = part[0] | part[1] | part[2] | part[3];
}

// Pass 2: one block per window sorts its rows by (mask, row) and replaces the masks by the row
// order.  Stable least-significant-digit radix sort of the permutation, 7 bits per pass
// (ceil(K / 7) passes): a warp owns 128 consecutive positions, ranks equal digits with
// match_any (lane order = position order, so the sort is stable and deterministic), the
// per-(digit, warp) counts are scanned digit-major by the block, and rows scatter to their place.
constexpr int kDigitBits = 7, kDigits = 1 << kDigitBits;

template <int kTileWindow>
__global__ void __launch_bounds__(kTileOrderThreads)
kmap_window_sort_kernel(int32_t* __restrict__ rows_io, int64_t M, int K) {
  extern __shared__ __align__(16) uint8_t sort_smem[];
  uint32_t* mask_s = reinterpret_cast<uint32_t*>(sort_smem);                       // mask of local row r (never moves)
  uint16_t (*perm_s)[kTileWindow] = reinterpret_cast<uint16_t (*)[kTileWindow]>(mask_s + kTileWindow);  // current / next order
  uint16_t* cnt = reinterpret_cast<uint16_t*>(perm_s + 2);                         // [digit][warp] counts, then start positions
  uint32_t* warp_sums = reinterpret_cast<uint32_t*>(cnt + kDigits * 32);
  constexpr int kBatches = kTileWindow / kTileOrderThreads;                        // rows per thread
  const int64_t base = (int64_t)blockIdx.x * kTileWindow;
  const int n = (int)min((int64_t)kTileWindow, M - base);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kTileWindow; i += kTileOrderThreads) {
    mask_s[i] = i < n ? (uint32_t)rows_io[base + i] : 0xFFFFFFFFu;  // padding sorts last (ties: stable)
    perm_s[0][i] = (uint16_t)i;
  }
  int cur = 0;
  const int passes = (K + kDigitBits - 1) / kDigitBits;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * kDigitBits;
    for (int i = threadIdx.x; i < kDigits * 32; i += kTileOrderThreads) cnt[i] = 0;
    __syncthreads();
    // rank inside (warp, digit); positions of a warp: warp * (32 * kBatches) + batch*32 + lane
    uint16_t row[kBatches];
    int dig[kBatches], rank[kBatches];
#pragma unroll
    for (int b = 0; b < kBatches; ++b) {
      row[b] = perm_s[cur][warp * (32 * kBatches) + b * 32 + lane];
      dig[b] = (int)((mask_s[row[b]] >> shift) & (kDigits - 1));
      const unsigned same = __match_any_sync(0xFFFFFFFFu, dig[b]);
      const int r = __popc(same & ((1u << lane) - 1u));
      const int leader = __ffs(same) - 1;
      int before = 0;
      if (r == 0) {  // the first lane of each digit updates the warp's count
        before = cnt[dig[b] * 32 + warp];
        cnt[dig[b] * 32 + warp] = (uint16_t)(before + __popc(same));
      }
      before = __shfl_sync(0xFFFFFFFFu, before, leader);
      rank[b] = before + r;
      __syncwarp();  // the next batch reads the counts written here
    }
    __syncthreads();
    // exclusive scan of the counts in (digit, warp) order: 4 consecutive entries per thread
    {
      constexpr int kPer = kDigits * 32 / kTileOrderThreads;
      uint32_t v[kPer], sum = 0;
#pragma unroll
      for (int j = 0; j < kPer; ++j) { v[j] = cnt[threadIdx.x * kPer + j]; sum += v[j]; }
      uint32_t incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += o;
      }
      if (lane == 31) warp_sums[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        const uint32_t w = warp_sums[lane];
        uint32_t wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, wi, d);
          if (lane >= d) wi += o;
        }
        warp_sums[lane] = wi - w;
      }
      __syncthreads();
      uint32_t run = warp_sums[warp] + incl - sum;
#pragma unroll
      for (int j = 0; j < kPer; ++j) { cnt[threadIdx.x * kPer + j] = (uint16_t)run; run += v[j]; }
    }
    __syncthreads();
#pragma unroll
    for (int b = 0; b < kBatches; ++b) perm_s[cur ^ 1][cnt[dig[b] * 32 + warp] + rank[b]] = row[b];
    cur ^= 1;
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += kTileOrderThreads) rows_io[base + i] = (int32_t)(base + perm_s[cur][i]);
}

// Pass 3: nbr_tiled[k][s] = nbr[k][out_rows[s]]; a block stages one window of one offset in
// shared memory, so global memory is read and written in full lines.
template <int kTileWindow>
__global__ void __launch_bounds__(kTileOrderThreads)
kmap_permute_kernel(const int32_t* __restrict__ nbr, const int32_t* __restrict__ out_rows, int64_t M, int K,
                    int32_t* __restrict__ nbr_tiled) {
  extern __shared__ __align__(16) uint8_t permute_smem[];
  int32_t* stage = reinterpret_cast<int32_t*>(permute_smem);
  uint16_t* perm = reinterpret_cast<uint16_t*>(stage + kTileWindow);
  const int64_t base = (int64_t)blockIdx.x * kTileWindow;
  const int n = (int)min((int64_t)kTileWindow, M - base);
  for (int i = threadIdx.x; i < n; i += kTileOrderThreads) perm[i] = (uint16_t)(out_rows[base + i] - base);
  const int k0 = blockIdx.y * kTileCopyOffsets;
  for (int k = k0; k < min(K, k0 + kTileCopyOffsets); ++k) {
    const int32_t* src = nbr + (int64_t)k * M + base;
    int32_t* dst = nbr_tiled + (int64_t)k * M + base;
    __syncthreads();  // perm written / previous offset's stage fully read
    for (int i = threadIdx.x; i < n; i += kTileOrderThreads) stage[i] = __ldg(&src[i]);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kTileOrderThreads) dst[i] = stage[perm[i]];
  }
}

// ------------------------------------------------------------------ Morton

__device__ __forceinline__ unsigned long long spread3(unsigned long long n) {
  n &= 0x1FFFFFull;
  n = (n | (n << 32)) & 0x001F00000000FFFFull;
  n = (n | (n << 16)) & 0x001F0000FF0000FFull;
  n = (n | (n << 8)) & 0x100F00F00F00F00Full;
  n = (n | (n << 4)) & 0x10C30C30C30C30C3ull;
  n = (n | (n << 2)) & 0x1249249249249249ull;
  return n;
}

__global__ void morton20_kernel(const int32_t* __restrict__ coords, int64_t n, int row_ints, int col0,
                                const int32_t* __restrict__ min_xyz, int64_t* __restrict__ codes) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int mx = min_xyz ? __ldg(&min_xyz[0]) : 0, my = min_xyz ? __ldg(&min_xyz[1]) : 0,
            mz = min_xyz ? __ldg(&min_xyz[2]) : 0;
  const int32_t* r = coords + i * row_ints + col0;
  const unsigned long long x = (unsigned long long)(uint32_t)(r[0] - mx);
  const unsigned long long y = (unsigned long long)(uint32_t)(r[1] - my);
  const unsigned long long z = (unsigned long long)(uint32_t)(r[2] - mz);
  codes[i] = (int64_t)(spread3(x) | (spread3(y) << 1) | (spread3(z) << 2));
}

inline unsigned grid_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads); }

// Passes 2 and 3 of the tile order for one window size (their shared memory is opted into once per device).
template <int W>
int tile_order_windows(const int32_t* nbr, int64_t num_out, int num_offsets, int32_t* out_rows, int32_t* nbr_tiled,
                       cudaStream_t st) {
  constexpr size_t sort_bytes = (size_t)W * 4 + 2 * (size_t)W * 2 + kDigits * 32 * 2 + 32 * 4;
  constexpr size_t permute_bytes = (size_t)W * 4 + (size_t)W * 2;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return WCN_ERR_INITIALIZATION;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kmap_window_sort_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sort_bytes) != cudaSuccess ||
        cudaFuncSetAttribute(kmap_permute_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)permute_bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      return WCN_ERR_INITIALIZATION;
    }
    configured[dev] = true;
  }
  const unsigned windows = (unsigned)((num_out + W - 1) / W);
  kmap_window_sort_kernel<W><<<windows, kTileOrderThreads, sort_bytes, st>>>(out_rows, num_out, num_offsets);
  dim3 grid(windows, (unsigned)((num_offsets + kTileCopyOffsets - 1) / kTileCopyOffsets));
  kmap_permute_kernel<W><<<grid, kTileOrderThreads, permute_bytes, st>>>(nbr, out_rows, num_out, num_offsets, nbr_tiled);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

}  // namespace

// ====================================================================== C ABI

extern "C" int wcn_hash_table_bytes(int64_t capacity, int64_t* bytes) {
  if (capacity <= 0 || !bytes) return WCN_ERR_INVALID_PARAMETERS;
  *bytes = capacity * 20 + 16;  // keys, values, duplicate flag
  return WCN_OK;
}

#define WCN_DISPATCH_HASH(method, CALL)                         \
  switch (method) {                                             \
    case WCN_HASH_FNV1A: { constexpr int HM = WCN_HASH_FNV1A; CALL; } break;  \
    case WCN_HASH_CITY: { constexpr int HM = WCN_HASH_CITY; CALL; } break;    \
    case WCN_HASH_MURMUR: { constexpr int HM = WCN_HASH_MURMUR; CALL; } break; \
    default: return WCN_ERR_INVALID_PARAMETERS;                 \
  }

static inline bool parse_stride(const int32_t* stride, int* sx, int* sy, int* sz) {
  *sx = *sy = *sz = 1;
  if (stride) {
    *sx = stride[0]; *sy = stride[1]; *sz = stride[2];
  }
  return *sx > 0 && *sy > 0 && *sz > 0;
}

extern "C" int wcn_hash_build(const int32_t* keys, int64_t n, const int32_t* stride, void* table,
                              int64_t capacity, int hash_method, const int32_t* skip_if, int32_t* dev_status,
                              void* stream) {
  int sx, sy, sz;
  if (!table || capacity <= 0 || capacity > 0x7FFFFFFFll || n < 0 || n > capacity || (n > 0 && !keys) ||
      !parse_stride(stride, &sx, &sy, &sz))
    return WCN_ERR_INVALID_PARAMETERS;
  if ((reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(keys) & 15))
    return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  int4* tkeys = reinterpret_cast<int4*>(table);
  int* tvals = reinterpret_cast<int*>(tkeys + capacity);
  hash_clear_kernel<<<grid_for(capacity), kThreads, 0, st>>>(tkeys, tvals, capacity, skip_if);
  if (n > 0) {
    WCN_DISPATCH_HASH(hash_method, (hash_insert_kernel<HM><<<grid_for(n), kThreads, 0, st>>>(
                                       keys, n, sx, sy, sz, tkeys, tvals, (uint32_t)capacity, dev_status, skip_if)));
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_hash_search(const void* table, int64_t capacity, int hash_method,
                               const int32_t* queries, int64_t num_queries, int32_t* results,
                               void* stream) {
  if (!table || capacity <= 0 || capacity > 0x7FFFFFFFll || num_queries < 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_queries == 0) return WCN_OK;
  if (!queries || !results || (reinterpret_cast<uintptr_t>(queries) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  const int4* tkeys = reinterpret_cast<const int4*>(table);
  const int* tvals = reinterpret_cast<const int*>(tkeys + capacity);
  WCN_DISPATCH_HASH(hash_method, (hash_search_kernel<HM><<<grid_for(num_queries), kThreads, 0, wcn_stream(stream)>>>(
                                     tkeys, tvals, (uint32_t)capacity, queries, num_queries, results)));
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_unique_workspace_bytes(int64_t n, int64_t* bytes) {
  if (n < 0 || !bytes) return WCN_ERR_INVALID_PARAMETERS;
  *bytes = ((2 * n + unique_nblk(n) + 16) * 4 + 255) / 256 * 256;
  return WCN_OK;
}

extern "C" int wcn_unique_mark(const int32_t* coords, int64_t n, const int32_t* stride, const void* table,
                               int64_t capacity, int hash_method, void* workspace, int64_t* num_unique,
                               void* stream) {
  int sx, sy, sz;
  if (!table || !workspace || !num_unique || n < 0 || capacity <= 0 || capacity > 0x7FFFFFFFll ||
      !parse_stride(stride, &sx, &sy, &sz))
    return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  UniqueWs w = unique_ws(workspace, n);
  if (n == 0) {
    cudaMemsetAsync(num_unique, 0, sizeof(int64_t), st);
    return WCN_OK;
  }
  if (!coords || (reinterpret_cast<uintptr_t>(coords) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  const int4* tkeys = reinterpret_cast<const int4*>(table);
  const int* tvals = reinterpret_cast<const int*>(tkeys + capacity);
  WCN_DISPATCH_HASH(hash_method, (unique_mark_kernel<HM><<<(unsigned)w.nblk, kThreads, 0, st>>>(
                                     coords, n, sx, sy, sz, tkeys, tvals, (uint32_t)capacity, w.rep, w.block_counts)));
  scan_rows_kernel<<<1, 1024, 0, st>>>(w.block_counts, w.nblk, w.total);
  store_total_kernel<<<1, 32, 0, st>>>(w.total, num_unique);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_unique_emit(const int32_t* coords, int64_t n, const int32_t* stride, void* workspace,
                               int32_t* out_coords, int32_t* unique_index, int32_t* parent, void* stream) {
  int sx, sy, sz;
  if (!workspace || n < 0 || !parse_stride(stride, &sx, &sy, &sz)) return WCN_ERR_INVALID_PARAMETERS;
  if (n == 0) return WCN_OK;
  if (!coords || !out_coords || (reinterpret_cast<uintptr_t>(out_coords) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  UniqueWs w = unique_ws(workspace, n);
  unique_emit_kernel<<<(unsigned)w.nblk, kThreads, 0, st>>>(coords, n, sx, sy, sz, w.rep, w.block_counts,
                                                          w.rank_of, out_coords, unique_index);
  if (parent) unique_parent_kernel<<<(unsigned)w.nblk, kThreads, 0, st>>>(n, w.rep, w.rank_of, parent);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_workspace_bytes(int64_t num_queries, int32_t num_offsets, int64_t* bytes) {
  if (num_queries < 0 || num_offsets <= 0 || !bytes) return WCN_ERR_INVALID_PARAMETERS;
  const int64_t nblk = (num_queries + kThreads - 1) / kThreads;
  *bytes = (((int64_t)num_offsets * nblk + num_offsets + 16) * 4 + 255) / 256 * 256;
  return WCN_OK;
}

extern "C" int wcn_kmap_search_dilated(const void* table, int64_t capacity, int hash_method,
                                       const int32_t* queries, int64_t num_queries, const int32_t* stride,
                                       const int32_t* kernel_size, const int32_t* dilation, const int32_t* center,
                                       int32_t num_offsets, int32_t* nbr, void* workspace, void* stream) {
  KernelGeom g;
  if (!table || !kernel_size || capacity <= 0 || capacity > 0x7FFFFFFFll || num_queries < 0 ||
      !parse_stride(stride, &g.sx, &g.sy, &g.sz) || !parse_stride(dilation, &g.dx, &g.dy, &g.dz))
    return WCN_ERR_INVALID_PARAMETERS;
  g.kx = kernel_size[0]; g.ky = kernel_size[1]; g.kz = kernel_size[2];
  if (g.kx <= 0 || g.ky <= 0 || g.kz <= 0) return WCN_ERR_INVALID_PARAMETERS;
  const int K = g.kx * g.ky * g.kz;
  if (num_offsets <= 0 || num_offsets > K || num_offsets > 65535) return WCN_ERR_INVALID_PARAMETERS;
  g.cx = (g.kx & 1) ? g.kx / 2 : 0;
  g.cy = (g.ky & 1) ? g.ky / 2 : 0;
  g.cz = (g.kz & 1) ? g.kz / 2 : 0;
  if (center) {
    g.cx = center[0]; g.cy = center[1]; g.cz = center[2];
  }
  if (num_queries == 0) return WCN_OK;
  if (!queries || !nbr || (reinterpret_cast<uintptr_t>(queries) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  const int4* tkeys = reinterpret_cast<const int4*>(table);
  const int* tvals = reinterpret_cast<const int*>(tkeys + capacity);
  dim3 grid(grid_for(num_queries), (unsigned)num_offsets);
  if (workspace) {
    WCN_DISPATCH_HASH(hash_method, (kmap_search_kernel<HM, true><<<grid, kThreads, 0, wcn_stream(stream)>>>(
                                       tkeys, tvals, (uint32_t)capacity, queries, num_queries, g, nbr,
                                       reinterpret_cast<int*>(workspace))));
  } else {
    WCN_DISPATCH_HASH(hash_method, (kmap_search_kernel<HM, false><<<grid, kThreads, 0, wcn_stream(stream)>>>(
                                       tkeys, tvals, (uint32_t)capacity, queries, num_queries, g, nbr, nullptr)));
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_search(const void* table, int64_t capacity, int hash_method, const int32_t* queries,
                               int64_t num_queries, const int32_t* stride, const int32_t* kernel_size,
                               int32_t num_offsets, int32_t* nbr, void* workspace, void* stream) {
  return wcn_kmap_search_dilated(table, capacity, hash_method, queries, num_queries, stride, kernel_size, nullptr,
                                 nullptr, num_offsets, nbr, workspace, stream);
}

extern "C" int wcn_kmap_search_self(const void* table, int64_t capacity, int hash_method, const int32_t* keys,
                                    int64_t num_keys, const int32_t* kernel_size, const int32_t* dilation,
                                    int32_t* nbr, void* stream) {
  KernelGeom g;
  if (!table || !kernel_size || capacity <= 0 || capacity > 0x7FFFFFFFll || num_keys < 0 || num_keys >= 0x7FFFFFFFll ||
      !parse_stride(dilation, &g.dx, &g.dy, &g.dz))
    return WCN_ERR_INVALID_PARAMETERS;
  g.sx = g.sy = g.sz = 1;
  g.kx = kernel_size[0]; g.ky = kernel_size[1]; g.kz = kernel_size[2];
  if (g.kx <= 0 || g.ky <= 0 || g.kz <= 0 || !(g.kx & 1) || !(g.ky & 1) || !(g.kz & 1)) return WCN_ERR_INVALID_PARAMETERS;
  const int K = g.kx * g.ky * g.kz;
  if (K > 65535) return WCN_ERR_INVALID_PARAMETERS;
  g.cx = g.kx / 2; g.cy = g.ky / 2; g.cz = g.kz / 2;
  if (num_keys == 0) return WCN_OK;
  if (!keys || !nbr || (reinterpret_cast<uintptr_t>(keys) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const int4* tkeys = reinterpret_cast<const int4*>(table);
  const int* tvals = reinterpret_cast<const int*>(tkeys + capacity);
  // rows of the mirrored half that nobody points at stay -1
  if (K > 1)
    cudaMemsetAsync(nbr + (int64_t)(K / 2 + 1) * num_keys, 0xFF, sizeof(int32_t) * (size_t)(K / 2) * (size_t)num_keys, st);
  dim3 grid(grid_for(num_keys), (unsigned)K);
  WCN_DISPATCH_HASH(hash_method, (kmap_search_self_kernel<HM><<<grid, kThreads, 0, st>>>(
                                     tkeys, tvals, (uint32_t)capacity, keys, num_keys, g, K, nbr)));
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_count(const int32_t* nbr, int64_t num_queries, int32_t num_offsets, void* workspace,
                              void* stream) {
  if (num_queries < 0 || num_offsets <= 0 || num_offsets > 65535 || !workspace) return WCN_ERR_INVALID_PARAMETERS;
  if (num_queries == 0) return WCN_OK;
  if (!nbr) return WCN_ERR_INVALID_PARAMETERS;
  dim3 grid(grid_for(num_queries), (unsigned)num_offsets);
  kmap_count_kernel<<<grid, kThreads, 0, wcn_stream(stream)>>>(nbr, num_queries, reinterpret_cast<int*>(workspace));
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

// ------------------------------------------------------------------ allocation-free variant
//
// Scratch for wcn_kmap_search_static: per-block hit counts [num_offsets][blocks] followed by
// the per-offset totals, the same layout wcn_kmap_search / wcn_kmap_scan keep in the
// caller's workspace.  It lives in the library image, so every GPU that loads the library
// holds these 4 MiB until the process exits.
constexpr int64_t kStaticScratchInts = 1 << 20;
static __device__ __align__(256) int g_kmap_static_scratch[kStaticScratchInts];

// In host code the array's name is only a handle; the device address has to be asked for,
// once per device, with that device current (the caller's stream must belong to it).  The
// per-device cache is atomic, so concurrent first calls from several host threads are safe:
// each resolves the same address.
static int* kmap_static_scratch_ptr() {
  static std::atomic<int*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int* p = cached[dev].load(std::memory_order_acquire);
  if (!p) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_kmap_static_scratch) != cudaSuccess || !ptr) {
      (void)cudaGetLastError();
      return nullptr;
    }
    p = static_cast<int*>(ptr);
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

extern "C" int wcn_kmap_search_static(const void* table, int64_t capacity, int hash_method,
                                      const int32_t* queries, int64_t num_queries, const int32_t* stride,
                                      const int32_t* kernel_size, int32_t num_offsets, int32_t* nbr,
                                      int32_t* offsets, void* stream) {
  if (num_queries < 0 || num_offsets <= 0 || !offsets) return WCN_ERR_INVALID_PARAMETERS;
  const int64_t nblk = (num_queries + kThreads - 1) / kThreads;
  if ((int64_t)num_offsets * nblk + num_offsets + 16 > kStaticScratchInts) return WCN_ERR_SCRATCH_TOO_SMALL;
  int* scratch = kmap_static_scratch_ptr();  // first call on a device resolves the address
  if (!scratch) return WCN_ERR_INITIALIZATION;
  // Nothing in the scratch has to start at zero: the search writes every count it later
  // reads, the scan writes every total.
  const int rc = wcn_kmap_search(table, capacity, hash_method, queries, num_queries, stride, kernel_size,
                                 num_offsets, nbr, scratch, stream);
  if (rc != WCN_OK) return rc;
  return wcn_kmap_scan(scratch, num_queries, num_offsets, offsets, stream);
}

extern "C" int wcn_kmap_scan(void* workspace, int64_t num_queries, int32_t num_offsets, int32_t* offsets,
                             void* stream) {
  if (!workspace || !offsets || num_queries < 0 || num_offsets <= 0) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const int64_t nblk = (num_queries + kThreads - 1) / kThreads;
  int* counts = reinterpret_cast<int*>(workspace);
  int* totals = counts + (int64_t)num_offsets * nblk;
  if (nblk == 0) {
    cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (num_offsets + 1), st);
    return WCN_OK;
  }
  scan_rows_kernel<<<(unsigned)num_offsets, 1024, 0, st>>>(counts, nblk, totals);
  offsets_from_totals_kernel<<<1, 32, 0, st>>>(totals, num_offsets, offsets);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_compact(const int32_t* nbr, int64_t num_queries, int32_t num_offsets,
                                const void* workspace, const int32_t* offsets, int32_t* in_maps,
                                int32_t* out_maps, void* stream) {
  if (!workspace || !offsets || num_queries < 0 || num_offsets <= 0 || num_offsets > 65535)
    return WCN_ERR_INVALID_PARAMETERS;
  if (num_queries == 0) return WCN_OK;
  if (!nbr || !in_maps || !out_maps) return WCN_ERR_INVALID_PARAMETERS;
  dim3 grid(grid_for(num_queries), (unsigned)num_offsets);
  kmap_compact_kernel<<<grid, kThreads, 0, wcn_stream(stream)>>>(nbr, num_queries,
                                                               reinterpret_cast<const int*>(workspace), offsets,
                                                               in_maps, out_maps);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_nbr_from_maps(const int32_t* in_maps, const int32_t* out_maps, const int32_t* offsets,
                                 int32_t num_offsets, int64_t num_pairs, int64_t num_out, int32_t* nbr,
                                 void* stream) {
  if (num_offsets <= 0 || num_pairs < 0 || num_out < 0 || !offsets) return WCN_ERR_INVALID_PARAMETERS;
  if (num_out == 0) return WCN_OK;
  if (!nbr) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  cudaMemsetAsync(nbr, 0xFF, sizeof(int32_t) * (size_t)num_offsets * (size_t)num_out, st);
  if (num_pairs > 0) {
    if (!in_maps || !out_maps) return WCN_ERR_INVALID_PARAMETERS;
    nbr_from_maps_kernel<<<grid_for(num_pairs), kThreads, 0, st>>>(in_maps, out_maps, offsets, num_offsets,
                                                                  num_pairs, num_out, nbr);
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_nbr_transpose(const int32_t* nbr_fwd, int32_t num_offsets, int64_t num_out, int64_t num_in,
                                 int32_t* nbr_t, void* stream) {
  if (num_offsets <= 0 || num_offsets > 65535 || num_out < 0 || num_in < 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_in == 0) return WCN_OK;
  if (!nbr_t) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  cudaMemsetAsync(nbr_t, 0xFF, sizeof(int32_t) * (size_t)num_offsets * (size_t)num_in, st);
  if (num_out > 0) {
    if (!nbr_fwd) return WCN_ERR_INVALID_PARAMETERS;
    dim3 grid(grid_for(num_out), (unsigned)num_offsets);
    nbr_transpose_kernel<<<grid, kThreads, 0, st>>>(nbr_fwd, num_out, num_in, nbr_t);
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_tile_order(const int32_t* nbr, int64_t num_out, int32_t num_offsets, int32_t* out_rows,
                                   int32_t* nbr_tiled, void* stream) {
  if (num_offsets <= 0 || num_offsets > 32 || num_out < 0 || num_out >= 0x7FFFFFFFll) return WCN_ERR_INVALID_PARAMETERS;
  if (num_out == 0) return WCN_OK;
  if (!nbr || !out_rows || !nbr_tiled || nbr == nbr_tiled) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  // out_rows first holds the masks (sort keys), then (window by window) the order
  kmap_row_mask_kernel<<<grid_for(num_out), kThreads, 0, st>>>(nbr, num_out, num_offsets, (uint32_t*)out_rows);
  if (num_out > kTileWindowSmall) return tile_order_windows<kTileWindowLarge>(nbr, num_out, num_offsets, out_rows, nbr_tiled, st);
  return tile_order_windows<kTileWindowSmall>(nbr, num_out, num_offsets, out_rows, nbr_tiled, st);
}

extern "C" int wcn_kmap_tile_masks(const int32_t* nbr, int64_t num_out, int32_t num_offsets, uint32_t* masks,
                                   void* stream) {
  if (num_offsets <= 0 || num_offsets > 32 || num_out < 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_out == 0) return WCN_OK;
  if (!nbr || !masks) return WCN_ERR_INVALID_PARAMETERS;
  kmap_tile_mask_kernel<<<(unsigned)((num_out + 127) / 128), 128, 0, wcn_stream(stream)>>>(nbr, num_out, num_offsets,
                                                                                          masks);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_morton20(const int32_t* coords, int64_t n, int32_t row_ints, int32_t col0,
                            const int32_t* min_xyz, int64_t* codes, void* stream) {
  if (n < 0 || row_ints < 3 || col0 < 0 || col0 + 3 > row_ints) return WCN_ERR_INVALID_PARAMETERS;
  if (n == 0) return WCN_OK;
  if (!coords || !codes) return WCN_ERR_INVALID_PARAMETERS;
  morton20_kernel<<<grid_for(n), kThreads, 0, wcn_stream(stream)>>>(coords, n, row_ints, col0, min_xyz, codes);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}
