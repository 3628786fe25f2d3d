// Kernel maps of Morton-ordered coordinate sets through a table of 4x4x4 bricks.
//
// A voxel-keyed hash table answers "which row holds (b, x, y, z)" with one random 32-byte
// sector per probe, 14..27 probes per output row: the search is bound by the L2 -> SM sector
// rate.  Rows sorted by Morton code (Voxels.sort) have more structure: the low six bits of a code
// are the voxel's position inside its 4x4x4 brick, so the rows of one brick are consecutive and
// ordered by that position.  One 32-byte entry per BRICK — key, 64-bit occupancy mask, first row
// — then answers every voxel of the brick:
//     row(b, x, y, z) = base + popcount(mask & below(bit(x, y, z)))       if the bit is set.
// A 3x3x3 (or 2x2x2) window touches at most 2x2x2 bricks, neighbouring output rows touch the
// same ones (L1 hits), and a thread that owns an output row resolves all its offsets from those
// eight entries and writes them with coalesced stores.  The table is about a twelfth of the voxel
// table on surface scans.
//
// Whether a coordinate set really is brick-ordered (with respect to the origin it is given) is
// decided on the device while the table is built; the search kernel falls back to probing the
// voxel table, offset by offset, when it is not, so the result is the same table either way and
// the host never has to ask.
#include "wcn_common.cuh"

namespace {

constexpr int kBrickThreads = 256;

struct __align__(32) BrickHeader {
  int32_t cap;         // slots in use (set while the table is cleared)
  int32_t valid;       // 1: every brick is one run of rows in strictly increasing position order
  int32_t num_bricks;
  int32_t reserved;
  int32_t origin[3];   // bricks are aligned to this corner
  int32_t pad;
};

struct __align__(32) BrickSlot {
  int4 key;                  // (batch, brick x, brick y, brick z); key.x == WCN_EMPTY_BATCH: empty
  unsigned long long mask;   // bit p set: the voxel at position p of the brick exists
  int32_t base;              // row of the brick's first voxel
  int32_t pad;
};

// Position of a voxel inside its brick = the low six bits of its Morton code (x in bit 0).
__device__ __forceinline__ uint32_t brick_pos(int x, int y, int z) {
  return (uint32_t)((x & 1) | ((y & 1) << 1) | ((z & 1) << 2) | ((x & 2) << 2) | ((y & 2) << 3) | ((z & 2) << 4));
}

__device__ __forceinline__ int4 brick_of(int4 c, int ox, int oy, int oz) {
  return make_int4(c.x, (c.y - ox) >> 2, (c.z - oy) >> 2, (c.w - oz) >> 2);  // arithmetic shift = floor
}

__device__ __forceinline__ uint32_t row_pos(int4 c, int ox, int oy, int oz) {
  return brick_pos((c.y - ox) & 3, (c.z - oy) & 3, (c.w - oz) & 3);
}

__host__ __device__ inline int64_t brick_cap_max(int64_t n) { return n * 2 > 64 ? n * 2 : 64; }

// Slots actually used: four per brick (a quarter full at most), within what was allocated.
__device__ __forceinline__ uint32_t brick_cap(int num_bricks, int64_t n) {
  int64_t want = (int64_t)num_bricks * 4;
  if (want < 64) want = 64;
  const int64_t cmax = brick_cap_max(n);
  return (uint32_t)(want < cmax ? want : cmax);
}

__device__ __forceinline__ uint32_t brick_slot(int4 key, uint32_t cap) {
  return wcn_slot(wcn_hash4<WCN_HASH_CITY>(key), cap);
}

// Pass 1: count the rows that start a brick; thread 0 also writes the header's constants.
__global__ void brick_count_kernel(const int32_t* __restrict__ keys, int64_t n, const int32_t* __restrict__ origin,
                                   BrickHeader* hdr) {
  const int ox = origin ? __ldg(&origin[0]) : 0, oy = origin ? __ldg(&origin[1]) : 0, oz = origin ? __ldg(&origin[2]) : 0;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int head = 0;
  if (i < n) {
    const int4 me = brick_of(__ldg(reinterpret_cast<const int4*>(keys) + i), ox, oy, oz);
    head = i == 0 || !wcn_key_eq(me, brick_of(__ldg(reinterpret_cast<const int4*>(keys) + i - 1), ox, oy, oz));
  }
  const int c = __syncthreads_count(head);
  if (threadIdx.x == 0 && c) atomicAdd(&hdr->num_bricks, c);
  if (i == 0) {
    hdr->valid = 1;
    hdr->origin[0] = ox; hdr->origin[1] = oy; hdr->origin[2] = oz;
  }
}

// Pass 2: empty the slots that will be used (their number follows from the brick count).
__global__ void brick_clear_kernel(BrickHeader* hdr, BrickSlot* slots, int64_t n) {
  const uint32_t cap = brick_cap(hdr->num_bricks, n);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) hdr->cap = (int32_t)cap;
  if (i < (int64_t)cap) {
    slots[i].key = make_int4(WCN_EMPTY_BATCH, 0, 0, 0);
    slots[i].mask = 0ull;
    slots[i].base = 0;
    slots[i].pad = 0;
  }
}

// Pass 3: the first row of every brick walks its run, checks the order, and inserts the brick.
__global__ void brick_insert_kernel(const int32_t* __restrict__ keys, int64_t n, BrickHeader* hdr, BrickSlot* slots) {
  const int ox = hdr->origin[0], oy = hdr->origin[1], oz = hdr->origin[2];
  const uint32_t cap = (uint32_t)hdr->cap;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4* rows = reinterpret_cast<const int4*>(keys);
  const int4 first = __ldg(rows + i);
  const int4 me = brick_of(first, ox, oy, oz);
  if (i > 0 && wcn_key_eq(me, brick_of(__ldg(rows + i - 1), ox, oy, oz))) return;  // not the first row of its brick
  if (first.x == WCN_EMPTY_BATCH) { hdr->valid = 0; return; }  // reserved batch value
  uint32_t last = row_pos(first, ox, oy, oz);
  unsigned long long mask = 1ull << last;
  for (int64_t j = i + 1; j < n && j < i + 65; ++j) {
    const int4 c = __ldg(rows + j);
    if (!wcn_key_eq(me, brick_of(c, ox, oy, oz))) break;
    const uint32_t p = row_pos(c, ox, oy, oz);
    if (p <= last) { hdr->valid = 0; return; }  // repeated voxel or rows not in Morton order
    mask |= 1ull << p;
    last = p;
  }
  const int4 empty = make_int4(WCN_EMPTY_BATCH, 0, 0, 0);
  uint32_t slot = brick_slot(me, cap);
  for (uint32_t probe = 0; probe < cap; ++probe) {
    int4* kp = &slots[slot].key;
    int4 cur = __ldcg(kp);
    if (cur.x == WCN_EMPTY_BATCH) {
      unsigned long long clo = ((unsigned long long)(uint32_t)empty.y << 32) | (uint32_t)empty.x;
      unsigned long long vlo = ((unsigned long long)(uint32_t)me.y << 32) | (uint32_t)me.x;
      unsigned long long vhi = ((unsigned long long)(uint32_t)me.w << 32) | (uint32_t)me.z;
      unsigned long long olo, ohi;
      asm volatile(
          "{\n\t.reg .b128 c, v, o;\n\t"
          "mov.b128 c, {%2, %3};\n\tmov.b128 v, {%4, %5};\n\t"
          "atom.global.relaxed.gpu.cas.b128 o, [%6], c, v;\n\t"
          "mov.b128 {%0, %1}, o;\n\t}"
          : "=l"(olo), "=l"(ohi)
          : "l"(clo), "l"(0ull), "l"(vlo), "l"(vhi), "l"(kp)
          : "memory");
      cur = make_int4((int)(uint32_t)olo, (int)(uint32_t)(olo >> 32), (int)(uint32_t)ohi, (int)(uint32_t)(ohi >> 32));
      if (cur.x == WCN_EMPTY_BATCH) {  // claimed: this thread alone writes the rest of the entry
        slots[slot].mask = mask;
        slots[slot].base = (int32_t)i;
        return;
      }
    }
    if (wcn_key_eq(cur, me)) { hdr->valid = 0; return; }  // the brick appears in two separate runs
    slot = slot + 1 == cap ? 0u : slot + 1;
  }
  hdr->valid = 0;  // no free slot (cannot happen at a quarter load, kept for safety)
}

// Entry of brick `key`, or mask 0 when there is no such brick.  Both halves of the 32-byte entry
// are requested together.
__device__ __forceinline__ void brick_lookup(const BrickSlot* __restrict__ slots, uint32_t cap, int4 key,
                                             unsigned long long* mask, int* base) {
  uint32_t slot = brick_slot(key, cap);
  *mask = 0ull;
  *base = 0;
  for (uint32_t probe = 0; probe < cap; ++probe) {
    const int4* e = reinterpret_cast<const int4*>(slots + slot);
    const int4 k = __ldg(e);
    const int4 v = __ldg(e + 1);
    if (k.x == WCN_EMPTY_BATCH) return;
    if (wcn_key_eq(k, key)) {
      *mask = ((unsigned long long)(uint32_t)v.y << 32) | (uint32_t)v.x;
      *base = v.z;
      return;
    }
    slot = slot + 1 == cap ? 0u : slot + 1;
  }
}

// One thread per output row: the window of the row (kx x ky x kz positions, each axis at most four
// wide, dilation 1) lies in at most 2 x 2 x 2 bricks; their entries are fetched once and every
// offset is answered from them.  nbr[k * M + m] as wcn_kmap_search writes it.
// KS: the window's width when it is the same along the three axes and known at compile time (2 or
// 3: the loops unroll and the positions inside a brick become constants), 0: kx, ky, kz as given.
template <int METHOD, int KS>
__global__ void __launch_bounds__(kBrickThreads)
kmap_search_bricks_kernel(const BrickHeader* __restrict__ hdr, const BrickSlot* __restrict__ slots,
                          const int4* __restrict__ tkeys, const int* __restrict__ tvals, uint32_t vcap,
                          const int32_t* __restrict__ queries, int64_t M, int sx, int sy, int sz, int kx_, int ky_,
                          int kz_, int32_t* __restrict__ nbr) {
  __shared__ unsigned long long s_mask[8][kBrickThreads];
  __shared__ int s_base[8][kBrickThreads];
  const int kx = KS ? KS : kx_, ky = KS ? KS : ky_, kz = KS ? KS : kz_;
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const int4 q = __ldg(reinterpret_cast<const int4*>(queries) + m);
  const int cx = (kx & 1) ? kx / 2 : 0, cy = (ky & 1) ? ky / 2 : 0, cz = (kz & 1) ? kz / 2 : 0;
  const int x0 = q.y * sx - cx, y0 = q.z * sy - cy, z0 = q.w * sz - cz;  // first position of the window
  if (!__ldg(&hdr->valid)) {
    // The rows were not brick-ordered: probe the voxel table position by position.
    for (int i = 0; i < kx; ++i)
      for (int j = 0; j < ky; ++j)
        for (int l = 0; l < kz; ++l)
          nbr[(int64_t)((i * ky + j) * kz + l) * M + m] =
              wcn_lookup<METHOD>(tkeys, tvals, vcap, make_int4(q.x, x0 + i, y0 + j, z0 + l));
    return;
  }
  const uint32_t cap = (uint32_t)__ldg(&hdr->cap);
  const int rx = x0 - __ldg(&hdr->origin[0]), ry = y0 - __ldg(&hdr->origin[1]), rz = z0 - __ldg(&hdr->origin[2]);
  const int bx0 = rx >> 2, by0 = ry >> 2, bz0 = rz >> 2;
  const bool two_x = ((rx + kx - 1) >> 2) > bx0, two_y = ((ry + ky - 1) >> 2) > by0, two_z = ((rz + kz - 1) >> 2) > bz0;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    const int ix = t & 1, iy = (t >> 1) & 1, iz = t >> 2;
    unsigned long long mk = 0ull;
    int bs = 0;
    if ((!ix || two_x) && (!iy || two_y) && (!iz || two_z))
      brick_lookup(slots, cap, make_int4(q.x, bx0 + ix, by0 + iy, bz0 + iz), &mk, &bs);
    s_mask[t][threadIdx.x] = mk;
    s_base[t][threadIdx.x] = bs;
  }
  int32_t* dst = nbr + m;  // offsets in the order (i, j, l), M apart
#pragma unroll
  for (int i = 0; i < kx; ++i) {
    const int x = rx + i, tx = (x >> 2) - bx0;
    const uint32_t px = brick_pos(x & 3, 0, 0);
#pragma unroll
    for (int j = 0; j < ky; ++j) {
      const int y = ry + j, txy = tx | (((y >> 2) - by0) << 1);
      const uint32_t pxy = px | brick_pos(0, y & 3, 0);
#pragma unroll
      for (int l = 0; l < kz; ++l, dst += M) {
        const int z = rz + l, t = txy | (((z >> 2) - bz0) << 2);
        const unsigned long long mk = s_mask[t][threadIdx.x];
        const uint32_t p = pxy | brick_pos(0, 0, z & 3);
        int found = -1;
        if ((mk >> p) & 1ull) found = s_base[t][threadIdx.x] + __popcll(mk & ((1ull << p) - 1ull));
        *dst = found;
      }
    }
  }
}

inline unsigned brick_grid(int64_t n) { return (unsigned)((n + kBrickThreads - 1) / kBrickThreads); }

}  // namespace

// Device address of the table's "usable" word, for wcn_hash_build's skip_if argument.
extern "C" const int32_t* wcn_brick_usable_flag(const void* brick_table) {
  return brick_table ? &reinterpret_cast<const BrickHeader*>(brick_table)->valid : nullptr;
}

extern "C" int wcn_brick_table_bytes(int64_t n, int64_t* bytes) {
  if (n < 0 || !bytes) return WCN_ERR_INVALID_PARAMETERS;
  *bytes = (int64_t)sizeof(BrickHeader) + brick_cap_max(n) * (int64_t)sizeof(BrickSlot);
  return WCN_OK;
}

extern "C" int wcn_brick_build(const int32_t* keys, int64_t n, const int32_t* origin, void* table, void* stream) {
  if (!table || n < 0 || n >= 0x3FFFFFFFll || (n > 0 && !keys)) return WCN_ERR_INVALID_PARAMETERS;
  if ((reinterpret_cast<uintptr_t>(table) & 31) || (reinterpret_cast<uintptr_t>(keys) & 15)) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  BrickHeader* hdr = reinterpret_cast<BrickHeader*>(table);
  BrickSlot* slots = reinterpret_cast<BrickSlot*>(hdr + 1);
  cudaMemsetAsync(hdr, 0, sizeof(BrickHeader), st);  // valid = 0 until the count pass has run
  if (n == 0) return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
  brick_count_kernel<<<brick_grid(n), kBrickThreads, 0, st>>>(keys, n, origin, hdr);
  brick_clear_kernel<<<brick_grid(brick_cap_max(n)), kBrickThreads, 0, st>>>(hdr, slots, n);
  brick_insert_kernel<<<brick_grid(n), kBrickThreads, 0, st>>>(keys, n, hdr, slots);
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_kmap_search_bricks(const void* brick_table, const void* table, int64_t capacity, int hash_method,
                                      const int32_t* queries, int64_t num_queries, const int32_t* stride,
                                      const int32_t* kernel_size, int32_t* nbr, void* stream) {
  if (!brick_table || !table || !kernel_size || capacity <= 0 || capacity > 0x7FFFFFFFll || num_queries < 0)
    return WCN_ERR_INVALID_PARAMETERS;
  int sx = 1, sy = 1, sz = 1;
  if (stride) { sx = stride[0]; sy = stride[1]; sz = stride[2]; }
  const int kx = kernel_size[0], ky = kernel_size[1], kz = kernel_size[2];
  if (sx <= 0 || sy <= 0 || sz <= 0 || kx <= 0 || ky <= 0 || kz <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (kx > 4 || ky > 4 || kz > 4) return WCN_ERR_UNSUPPORTED_CONFIG;  // a wider window spans three bricks
  if (num_queries == 0) return WCN_OK;
  if (!queries || !nbr || (reinterpret_cast<uintptr_t>(queries) & 15) || (reinterpret_cast<uintptr_t>(brick_table) & 31))
    return WCN_ERR_INVALID_PARAMETERS;
  const BrickHeader* hdr = reinterpret_cast<const BrickHeader*>(brick_table);
  const BrickSlot* slots = reinterpret_cast<const BrickSlot*>(hdr + 1);
  const int4* tkeys = reinterpret_cast<const int4*>(table);
  const int* tvals = reinterpret_cast<const int*>(tkeys + capacity);
  cudaStream_t st = wcn_stream(stream);
  const int ks = (kx == ky && ky == kz && (kx == 2 || kx == 3)) ? kx : 0;
#define WCN_BRICK_LAUNCH(HM, KS)                                                                                    \
  kmap_search_bricks_kernel<HM, KS><<<brick_grid(num_queries), kBrickThreads, 0, st>>>(                             \
      hdr, slots, tkeys, tvals, (uint32_t)capacity, queries, num_queries, sx, sy, sz, kx, ky, kz, nbr)
#define WCN_BRICK_CASE(HM)                                                                                          \
  case HM:                                                                                                          \
    if (ks == 3) WCN_BRICK_LAUNCH(HM, 3);                                                                           \
    else if (ks == 2) WCN_BRICK_LAUNCH(HM, 2);                                                                      \
    else WCN_BRICK_LAUNCH(HM, 0);                                                                                   \
    break;
  switch (hash_method) {
    WCN_BRICK_CASE(WCN_HASH_FNV1A)
    WCN_BRICK_CASE(WCN_HASH_CITY)
    WCN_BRICK_CASE(WCN_HASH_MURMUR)
    default: return WCN_ERR_INVALID_PARAMETERS;
  }
#undef WCN_BRICK_CASE
#undef WCN_BRICK_LAUNCH
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}
