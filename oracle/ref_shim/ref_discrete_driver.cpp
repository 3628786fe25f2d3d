// Sequential host driver around the reference's kernel-map kernels
// (warpconvnet/csrc/discrete_kernels.cu).  REF_SRC is the absolute path of that
// file, given on the compiler command line; its text is never copied.
#include "cuda_cpu_shim.h"
#include REF_SRC

// found[k * M + m] for every kernel position k of a kx*ky*kz window, exactly as
// launched by _kernel_map_from_size (torch_discrete.py:318-331): 2-D grid of
// (ceil(M/128), ceil(K/8)) blocks of (128, 8) threads.
extern "C" int ref_kernel_map_size_4d(const int* table_kvs, const int* keys, const int* queries,
                                      const int* kernel_sizes, int* found, int num_queries,
                                      int capacity, int num_kernels, int hash_method) {
  const int tx = 128, ty = 8;
  blockDim = {(unsigned)tx, (unsigned)ty, 1};
  unsigned gx = (num_queries + tx - 1) / tx, gy = (num_kernels + ty - 1) / ty;
  gridDim = {gx, gy, 1};
  for (unsigned by = 0; by < gy; ++by)
    for (unsigned bx = 0; bx < gx; ++bx) {
      blockIdx = {bx, by, 0};
      for (unsigned y = 0; y < (unsigned)ty; ++y)
        for (unsigned x = 0; x < (unsigned)tx; ++x) {
          threadIdx = {x, y, 0};
          switch (hash_method) {
            case 0: kernel_map_size_4d_fnv1a(table_kvs, keys, queries, kernel_sizes, found, num_queries, capacity, num_kernels); break;
            case 1: kernel_map_size_4d_city(table_kvs, keys, queries, kernel_sizes, found, num_queries, capacity, num_kernels); break;
            case 2: kernel_map_size_4d_murmur(table_kvs, keys, queries, kernel_sizes, found, num_queries, capacity, num_kernels); break;
            default: return -1;
          }
        }
    }
  return 0;
}

// Compaction kernel launched as in _kernel_map_search_to_result
// (torch_discrete.py:126-149): one thread per element of found[K, M].
extern "C" int ref_map_found_indices_to_maps(const int* found, const int* mapped_indices,
                                             const int* offsets, int* in_maps, int* out_maps,
                                             int num_kernels, int num_queries) {
  long long total = (long long)num_kernels * num_queries;
  const int threads = 256;
  blockDim = {(unsigned)threads, 1, 1};
  long long blocks = (total + threads - 1) / threads;
  gridDim = {(unsigned)blocks, 1, 1};
  for (long long b = 0; b < blocks; ++b) {
    blockIdx = {(unsigned)b, 0, 0};
    for (int t = 0; t < threads; ++t) {
      threadIdx = {(unsigned)t, 0, 0};
      map_found_indices_to_maps_cuda(found, mapped_indices, offsets, in_maps, out_maps, num_kernels, num_queries);
    }
  }
  return 0;
}

// found[k * M + m] for an explicit list of kernel offsets [K, key_dim] (batch column first),
// exactly as launched by _kernel_map_from_offsets (torch_discrete.py:160-241): 2-D grid of
// (ceil(M/128), ceil(K/8)) blocks of (128, 8) threads.  This is the reference's path for
// dilated windows and custom window centres.
extern "C" int ref_kernel_map_offset(const int* table_kvs, const int* keys, const int* queries,
                                     const int* kernel_offsets, int* found, int num_queries, int key_dim,
                                     int num_offsets, int capacity, int hash_method) {
  const int tx = 128, ty = 8;
  blockDim = {(unsigned)tx, (unsigned)ty, 1};
  unsigned gx = (num_queries + tx - 1) / tx, gy = (num_offsets + ty - 1) / ty;
  gridDim = {gx, gy, 1};
  for (unsigned by = 0; by < gy; ++by)
    for (unsigned bx = 0; bx < gx; ++bx) {
      blockIdx = {bx, by, 0};
      for (unsigned y = 0; y < (unsigned)ty; ++y)
        for (unsigned x = 0; x < (unsigned)tx; ++x) {
          threadIdx = {x, y, 0};
          switch (hash_method) {
            case 0: kernel_map_offset_fnv1a(table_kvs, keys, queries, kernel_offsets, found, num_queries, key_dim, num_offsets, capacity); break;
            case 1: kernel_map_offset_city(table_kvs, keys, queries, kernel_offsets, found, num_queries, key_dim, num_offsets, capacity); break;
            case 2: kernel_map_offset_murmur(table_kvs, keys, queries, kernel_offsets, found, num_queries, key_dim, num_offsets, capacity); break;
            default: return -1;
          }
        }
    }
  return 0;
}
