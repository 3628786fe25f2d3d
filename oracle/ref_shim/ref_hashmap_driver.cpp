// Sequential host driver around the reference's hash-table kernels
// (warpconvnet/csrc/hashmap_kernels.cu).  REF_SRC is the absolute path of that
// file, given on the compiler command line; its text is never copied.
#include "cuda_cpu_shim.h"
#include REF_SRC

namespace {
template <typename F>
void launch_1d(long long n, int threads, F body) {
  blockDim = {(unsigned)threads, 1, 1};
  long long blocks = (n + threads - 1) / threads;
  gridDim = {(unsigned)blocks, 1, 1};
  for (long long b = 0; b < blocks; ++b) {
    blockIdx = {(unsigned)b, 0, 0};
    for (int t = 0; t < threads; ++t) {
      threadIdx = {(unsigned)t, 0, 0};
      body();
    }
  }
}
}  // namespace

// hash_method: 0 = fnv1a, 1 = city, 2 = murmur (order of HashMethod in
// warpconvnet/geometry/coords/search/torch_hashmap.py:17-32).
extern "C" int ref_hash_insert(int* table_kvs, const int* keys, int num_keys, int key_dim,
                               int capacity, int hash_method) {
  launch_1d(capacity, 256, [&] { prepare_key_value_pairs_kernel(table_kvs, capacity); });
  switch (hash_method) {
    case 0: launch_1d(num_keys, 256, [&] { insert_kernel_fnv1a(table_kvs, keys, num_keys, key_dim, capacity); }); break;
    case 1: launch_1d(num_keys, 256, [&] { insert_kernel_city(table_kvs, keys, num_keys, key_dim, capacity); }); break;
    case 2: launch_1d(num_keys, 256, [&] { insert_kernel_murmur(table_kvs, keys, num_keys, key_dim, capacity); }); break;
    default: return -1;
  }
  return 0;
}

extern "C" int ref_hash_search(const int* table_kvs, const int* keys, const int* queries,
                               int* results, int num_queries, int key_dim, int capacity,
                               int hash_method) {
  switch (hash_method) {
    case 0: launch_1d(num_queries, 256, [&] { search_kernel_fnv1a(table_kvs, keys, queries, results, num_queries, key_dim, capacity); }); break;
    case 1: launch_1d(num_queries, 256, [&] { search_kernel_city(table_kvs, keys, queries, results, num_queries, key_dim, capacity); }); break;
    case 2: launch_1d(num_queries, 256, [&] { search_kernel_murmur(table_kvs, keys, queries, results, num_queries, key_dim, capacity); }); break;
    default: return -1;
  }
  return 0;
}
