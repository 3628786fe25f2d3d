/*
 * wcn_b200.h — C ABI of libwcn_b200.so: the sm_100a kernels behind the sparse-convolution
 * hot path (coordinate hash table, kernel-map generation, stride-2 coordinate
 * down-sampling, Morton code, gather-GEMM-scatter convolution with a fused
 * BatchNorm/ReLU/residual epilogue).
 *
 * Conventions
 *  - plain C: device pointers, 64-bit sizes, enum codes; no C++ or torch types.
 *  - every entry point returns an int status (WCN_OK or a negative wcn_status code) and
 *    never throws, exits or allocates device memory: outputs and scratch are passed in,
 *    with a *_bytes query where the size is not obvious.
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call
 *    returns without synchronising.
 *  - conditions that can only be detected on the device (hash-table overflow, a bounded
 *    wait that ran out, an index that names no row) are reported through `dev_status`, a
 *    device int32 the caller zeroes beforehand and must read back (poll) when it wants to
 *    know: kernels only ever store a negative wcn_status code into it and it stays set until
 *    the caller zeroes it again.  WCN_ERR_WAIT_EXPIRED overrides the others (the kernel that
 *    stored it gave up half-way): while the word holds it the tensor-core kernels do no work, a
 *    convolution fills the rows it was asked for with NaN and a weight gradient adds nothing.
 *    An out-of-range index is never followed: the access is skipped (the neighbour counts as
 *    absent), the rest of the launch is computed normally and WCN_ERR_BOUNDS is stored if the
 *    word was clean.
 *  - the device the stream belongs to must be the current device of the calling thread
 *    (launch geometry is taken from the current device's properties).
 *  - coordinates are int32 rows (batch, x, y, z).  The batch value INT32_MIN is reserved
 *    (it marks an empty hash slot).
 *
 * Each declaration names the reference interface it replaces (paths relative to the
 * reference project root).
 */
#ifndef WCN_B200_H_
#define WCN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  -1..-5 mirror the reference's GemmStatus
 * (warpconvnet/csrc/include/gemm_error_codes.h:5-13); the rest are new. */
enum wcn_status {
  WCN_OK = 0,
  WCN_ERR_PROBLEM_NOT_SUPPORTED = -1,
  WCN_ERR_INITIALIZATION = -2,
  WCN_ERR_EXECUTION = -3,
  WCN_ERR_UNSUPPORTED_CONFIG = -4,
  WCN_ERR_INVALID_PARAMETERS = -5,
  WCN_ERR_HASH_OVERFLOW = -6,
  WCN_ERR_WAIT_EXPIRED = -7,
  WCN_ERR_BOUNDS = -8,
  WCN_ERR_SCRATCH_TOO_SMALL = -9
};

/* Element types of feature / weight tensors. */
enum wcn_dtype { WCN_F32 = 0, WCN_F16 = 1, WCN_BF16 = 2 };

/* Hash functions, in the order of HashMethod
 * (warpconvnet/geometry/coords/search/torch_hashmap.py:17-32). */
enum wcn_hash_method { WCN_HASH_FNV1A = 0, WCN_HASH_CITY = 1, WCN_HASH_MURMUR = 2 };

/* Reductions of wcn_row_reduce, the native part of REDUCTIONS (warpconvnet/ops/reductions.py:13-21). */
enum wcn_reduce_op { WCN_REDUCE_MIN = 0, WCN_REDUCE_MAX = 1, WCN_REDUCE_SUM = 2, WCN_REDUCE_MEAN = 3, WCN_REDUCE_MUL = 4 };

/* Convolution kernels selectable through wcn_conv_fwd's `algo`. */
enum wcn_conv_algo { WCN_CONV_AUTO = 0, WCN_CONV_SIMT = 1, WCN_CONV_TCGEN05 = 2 };

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int wcn_version(void);

/* Human-readable text of a status code.
 * Replaces gemm_status_to_string (warpconvnet/csrc/warpconvnet_pybind.cpp:1220-1226). */
const char* wcn_status_string(int status);

/* ------------------------------------------------------------------ hash table */

/* Bytes of the table buffer for `capacity` slots (16-byte key + 4-byte value per slot, and a
 * 16-byte tail whose first word records whether a key was inserted twice).
 * Replaces the `[capacity, 2] int32` allocation in TorchHashTable.insert
 * (warpconvnet/geometry/coords/search/torch_hashmap.py:142). */
int wcn_hash_table_bytes(int64_t capacity, int64_t* bytes);

/* Clear the table and insert keys[n,4]; the value of a key is its row index (the smallest
 * one when a key occurs more than once).  stride = {sx,sy,sz} floor-divides x,y,z before
 * insertion ({1,1,1} or NULL: keys as given).  Needs n <= capacity.
 * skip_if (device int32, may be NULL): when it holds a non-zero value at the time the kernels run,
 * they do nothing and the table is left unbuilt — for a table that only backs up a brick table
 * (pass wcn_brick_usable_flag(brick_table), built earlier on the same stream): it is filled exactly
 * when wcn_kmap_search_bricks will need it.  A caller that later wants to probe the table itself
 * builds it again with skip_if = NULL.
 * Replaces prepare_key_value_pairs_kernel + insert_kernel_{fnv1a,city,murmur}
 * (warpconvnet/csrc/hashmap_kernels.cu:182-234, 258-270). */
int wcn_hash_build(const int32_t* keys, int64_t n, const int32_t* stride, void* table,
                   int64_t capacity, int hash_method, const int32_t* skip_if, int32_t* dev_status, void* stream);

/* results[i] = value of queries[i] in the table, or -1.
 * Replaces search_kernel_{fnv1a,city,murmur} (warpconvnet/csrc/hashmap_kernels.cu:237-301). */
int wcn_hash_search(const void* table, int64_t capacity, int hash_method, const int32_t* queries,
                    int64_t num_queries, int32_t* results, void* stream);

/* ------------------------------------------------------------------ distinct / strided coordinates */

/* Scratch bytes for wcn_unique_mark / wcn_unique_emit over n rows. */
int wcn_unique_workspace_bytes(int64_t n, int64_t* bytes);

/* Phase 1: with the table built by wcn_hash_build over the same (coords, stride), mark the
 * first occurrence of every distinct row of floor(coords / [1,sx,sy,sz]) and count them
 * into num_unique (device int64).
 * Replaces TorchHashTable.unique_index (torch_hashmap.py:303-322: search of all keys
 * followed by torch.unique) as used by stride_coords
 * (warpconvnet/geometry/coords/ops/stride.py:41-43). */
int wcn_unique_mark(const int32_t* coords, int64_t n, const int32_t* stride, const void* table,
                    int64_t capacity, int hash_method, void* workspace, int64_t* num_unique,
                    void* stream);

/* Phase 2 (after the caller has read num_unique and sized the outputs): write the distinct
 * rows in first-occurrence order to out_coords[num_unique,4], their source rows to
 * unique_index[num_unique], and for every input row the output row it collapsed into to
 * parent[n].  unique_index / parent may be NULL.
 * Replaces the gather `discretized_coords[unique_indices]` and the batch argsort of
 * stride_coords (stride.py:43-48); the order produced here is deterministic. */
int wcn_unique_emit(const int32_t* coords, int64_t n, const int32_t* stride, void* workspace,
                    int32_t* out_coords, int32_t* unique_index, int32_t* parent, void* stream);

/* ------------------------------------------------------------------ kernel map */

/* Scratch bytes for the three kernel-map calls (per-block hit counts). */
int wcn_kmap_workspace_bytes(int64_t num_queries, int32_t num_offsets, int64_t* bytes);

/* nbr[k*M + m] = row of (b, x*sx + i - cx, y*sy + j - cy, z*sz + l - cz) in the table or
 * -1, for k = (i*ky + j)*kz + l and c = size/2 for odd sizes, 0 for even sizes; also the
 * per-block hit counts in `workspace` (NULL: no counts; wcn_kmap_count makes them later if a
 * compact map is ever asked for).  num_offsets limits k to the first num_offsets
 * positions (the reference's skip_symmetric mode passes K/2).
 * Replaces kernel_map_size_4d_{fnv1a,city,murmur}
 * (warpconvnet/csrc/discrete_kernels.cu:264-334, 339-370). */
int wcn_kmap_search(const void* table, int64_t capacity, int hash_method, const int32_t* queries,
                    int64_t num_queries, const int32_t* stride, const int32_t* kernel_size,
                    int32_t num_offsets, int32_t* nbr, void* workspace, void* stream);

/* offsets[k] = number of hits of all offsets < k (device int32 [num_offsets+1]); turns the
 * per-block counts in `workspace` into write positions.
 * Replaces the cumsum/max/cumsum chain of _kernel_map_search_to_result
 * (warpconvnet/geometry/coords/search/torch_discrete.py:103-119). */
int wcn_kmap_scan(void* workspace, int64_t num_queries, int32_t num_offsets, int32_t* offsets,
                  void* stream);

/* wcn_kmap_search with dilated windows and a free window centre: position (i, j, l) of the
 * window probes x*sx + (i - cx)*dx and so on; `dilation` NULL means 1, `center` = {cx,cy,cz}
 * NULL means the default centre (size/2 for odd sizes, 0 for even sizes).
 * Replaces kernel_offsets_from_size with a kernel_dilation / center_offset and the offset-list
 * search _kernel_map_from_offsets (warpconvnet/geometry/coords/search/torch_discrete.py:44-77, 160-241). */
int wcn_kmap_search_dilated(const void* table, int64_t capacity, int hash_method, const int32_t* queries,
                            int64_t num_queries, const int32_t* stride, const int32_t* kernel_size,
                            const int32_t* dilation, const int32_t* center, int32_t num_offsets, int32_t* nbr,
                            void* workspace, void* stream);

/* wcn_kmap_search followed by wcn_kmap_scan, for callers that must not allocate device
 * memory.  Some hosts of this library cannot call cudaMalloc around it: plugins that are
 * handed a fixed arena by their framework and own no allocator, serving loops whose latency
 * budget forbids allocator calls (cudaMalloc synchronises the device), processes whose
 * memory pool is already exhausted or too fragmented for one more block.  For them the
 * per-block hit counts live in a fixed 4 MiB array inside the library image instead of a
 * caller-supplied workspace; the caller passes only inputs (table, queries) and outputs
 * (nbr[num_offsets * num_queries], offsets[num_offsets + 1], both device memory).
 * Limit: num_offsets * ceil(num_queries / 256) + num_offsets + 16 <= 1048576 (about 9.9 M
 * queries for a 3x3x3 window); larger problems return WCN_ERR_SCRATCH_TOO_SMALL and launch
 * nothing.  The entry point calls no allocator of any kind.  The first call on a device
 * looks up the array's device address (cudaGetSymbolAddress) for the CURRENT device, so the
 * device that owns `stream` must be current in the calling thread; make that first call before
 * any stream capture begins (concurrent first calls from several host threads are safe).  The
 * scanned hit counts stay inside the library, so this call yields the dense table and the
 * per-offset totals only: a caller that also wants the compact (in, out) lists runs
 * wcn_kmap_count + wcn_kmap_scan + wcn_kmap_compact with a workspace of its own.  All calls on a device share the one array and it keeps the last
 * call's contents (nothing in it needs clearing between calls), so two calls whose kernels
 * overlap on the GPU — different streams, no ordering between them — race; serialise them.
 * Every GPU that loads the library holds the array until the process exits.
 * No counterpart in the reference (its kernel-map path allocates through CuPy / torch on
 * every call, warpconvnet/geometry/coords/search/torch_discrete.py:312-315, 103-124). */
int wcn_kmap_search_static(const void* table, int64_t capacity, int hash_method,
                           const int32_t* queries, int64_t num_queries, const int32_t* stride,
                           const int32_t* kernel_size, int32_t num_offsets, int32_t* nbr,
                           int32_t* offsets, void* stream);

/* Compact nbr into in_maps / out_maps (length offsets[num_offsets]); within one offset the
 * pairs are in ascending output row.
 * Replaces map_found_indices_to_maps_cuda (warpconvnet/csrc/discrete_kernels.cu:183-213, 250-259). */
int wcn_kmap_compact(const int32_t* nbr, int64_t num_queries, int32_t num_offsets,
                     const void* workspace, const int32_t* offsets, int32_t* in_maps,
                     int32_t* out_maps, void* stream);

/* Dense neighbour table from a compact map: nbr[k*M + out_maps[p]] = in_maps[p] for
 * offsets[k] <= p < offsets[k+1], -1 elsewhere.  Requires out_maps to be distinct within
 * one offset (true of every map the reference builds).
 * Replaces nothing directly: the reference's kernels consume the compact lists
 * (warpconvnet/nn/functional/sparse_conv.py:300-310); this is the layout the
 * output-stationary convolution reads. */
int wcn_nbr_from_maps(const int32_t* in_maps, const int32_t* out_maps, const int32_t* offsets,
                      int32_t num_offsets, int64_t num_pairs, int64_t num_out, int32_t* nbr,
                      void* stream);

/* Neighbour table of the transposed map: nbr_t[k*num_in + i] = m wherever
 * nbr_fwd[k*num_out + m] = i, -1 elsewhere.  Requires each input row to occur at most once
 * per offset (true of every map the reference builds).
 * Replaces the in/out swap `IntSearchResult(in_maps=fwd.out_maps, out_maps=fwd.in_maps, ...)`
 * of transposed convolutions (warpconvnet/nn/functional/sparse_conv.py:1934-1938, 1953-1957). */
int wcn_nbr_transpose(const int32_t* nbr_fwd, int32_t num_offsets, int64_t num_out, int64_t num_in,
                      int32_t* nbr_t, void* stream);

/* Kernel map of a coordinate set onto itself: `keys` are the rows the table was built from
 * (same order), the window is odd (dilated by `dilation`, NULL = 1) and the stride 1, so nbr is [K, num_keys] with
 * K = kx*ky*kz.  Same result as wcn_kmap_search on those arguments.  When the keys are
 * distinct (the table records whether they are) the map is symmetric, nbr[k][m] = i exactly
 * when nbr[K-1-k][i] = m, and only the first half of the offsets and the centre are probed.
 * Leaves no hit counts.
 * Replaces kernel_map_size_4d_* for the submanifold case, i.e. what the reference's
 * skip_symmetric_kernel_map flag hints at (warpconvnet/geometry/coords/search/torch_discrete.py:291-296)
 * but never completes into the full map. */
int wcn_kmap_search_self(const void* table, int64_t capacity, int hash_method, const int32_t* keys,
                         int64_t num_keys, const int32_t* kernel_size, const int32_t* dilation, int32_t* nbr,
                         void* stream);

/* Bytes of the brick table of a coordinate set of n rows (a 32-byte header and one 32-byte entry
 * per slot, 2 n slots allocated, four per brick used). */
int wcn_brick_table_bytes(int64_t n, int64_t* bytes);

/* Brick table of keys[n,4]: one entry per 4x4x4 brick (aligned to `origin`, a DEVICE pointer to
 * three int32, NULL = 0) holding the brick's 64-bit occupancy mask and the row of its first voxel.
 * It is usable when the rows of every brick are consecutive and in Morton order inside the brick
 * — what sorting by the Morton code of (coords - origin) gives (Voxels.sort) — and the rows are
 * distinct; the build checks that on the device and marks the table unusable otherwise, in
 * which case wcn_kmap_search_bricks answers from the voxel table instead.  No host
 * synchronisation.
 * No counterpart in the reference, whose kernel map probes one voxel key per offset
 * (warpconvnet/csrc/discrete_kernels.cu:264-334) whatever the order of the rows; the ordering
 * itself is the reference's (warpconvnet/geometry/types/voxels.py:255-267,
 * warpconvnet/csrc/morton_code.cu:15-22). */
int wcn_brick_build(const int32_t* keys, int64_t n, const int32_t* origin, void* table, void* stream);

/* Device address of the word of a brick table that is non-zero when the table is usable (valid
 * after wcn_brick_build has run on the stream); what wcn_hash_build takes as skip_if.  Host-only,
 * launches nothing.  No counterpart in the reference. */
const int32_t* wcn_brick_usable_flag(const void* brick_table);

/* wcn_kmap_search (same nbr[k*M + m], same offset order and centre rule, dilation 1) answered
 * from a brick table: one thread per query fetches the at most 2x2x2 brick entries its window
 * touches and resolves every offset from them.  Window sizes up to 4 per axis
 * (WCN_ERR_UNSUPPORTED_CONFIG beyond).  `table` / `capacity` / `hash_method` are the voxel table
 * of the same keys (wcn_hash_build), used when the brick table was marked unusable.
 * Replaces kernel_map_size_4d_{fnv1a,city,murmur}
 * (warpconvnet/csrc/discrete_kernels.cu:264-334, 339-370) for Morton-ordered inputs. */
int wcn_kmap_search_bricks(const void* brick_table, const void* table, int64_t capacity, int hash_method,
                           const int32_t* queries, int64_t num_queries, const int32_t* stride,
                           const int32_t* kernel_size, int32_t* nbr, void* stream);

/* Per-block hit counts of a dense neighbour table into `workspace`, exactly what
 * wcn_kmap_search leaves there; for maps that were searched without counts.
 * Replaces the `found >= 0` pass of map_found_indices_to_maps_cuda
 * (warpconvnet/csrc/discrete_kernels.cu:183-213). */
int wcn_kmap_count(const int32_t* nbr, int64_t num_queries, int32_t num_offsets, void* workspace,
                   void* stream);

/* Tile order of a neighbour table: within each window of consecutive output rows (4096 rows for
 * tables of at most 4096 rows, else 16384) the rows are sorted by their neighbour-presence key (a
 * bit per offset, set when nbr[k][m] >= 0; for 27 offsets the centre of the 3x3x3 window is bit 0,
 * then the face, edge and corner offsets, so the rarest ones are the most significant; otherwise bit
 * k; ties by row), so that rows with the same present offsets share a 128-row tile and the
 * convolution skips the (tile, offset) pairs that have no neighbour at all.
 *   out_rows[s]        the output row that slot s of the tiled table stands for (a permutation
 *                      of 0..num_out-1 that moves no row out of its window)
 *   nbr_tiled[k][s]    = nbr[k][out_rows[s]]
 * Pass both to wcn_conv_fwd (nbr = nbr_tiled, out_rows = out_rows); the results are bit
 * identical to the untiled call.  num_offsets <= 32.  Deterministic.
 * No reference counterpart: the reference's implicit GEMM walks per-offset pair lists
 * (warpconvnet/nn/functional/sparse_conv.py:300-310) and never forms output tiles. */
int wcn_kmap_tile_order(const int32_t* nbr, int64_t num_out, int32_t num_offsets, int32_t* out_rows,
                        int32_t* nbr_tiled, void* stream);

/* masks[t] = set of offsets k (bit k) for which some row of [128 t, 128 t + 128) has nbr[k][row] >= 0;
 * ceil(num_out / 128) words, num_offsets <= 32.  Lets a kernel that walks the table in 128-row
 * steps (wcn_conv_wgrad) skip the steps that cannot contribute.  No reference counterpart. */
int wcn_kmap_tile_masks(const int32_t* nbr, int64_t num_out, int32_t num_offsets, uint32_t* masks,
                        void* stream);

/* ------------------------------------------------------------------ Morton code */

/* codes[i] = 3-D Morton code of (x - min_xyz[0], y - min_xyz[1], z - min_xyz[2]), x in bit
 * 0, y in bit 1, z in bit 2, up to 21 bits per axis.  coords has `row_ints` int32 per row
 * and the x column at `col0` (3,0 for xyz rows; 4,1 for batch-indexed rows).  `min_xyz` is a
 * DEVICE pointer to three int32 (or NULL for no shift), so the caller's min-reduction needs
 * no round trip to the host.
 * Replaces assign_order_discrete_20bit_kernel_4points (warpconvnet/csrc/morton_code.cu:71-94)
 * and the min subtraction of morton_code (coords/ops/serialization.py:224-225). */
int wcn_morton20(const int32_t* coords, int64_t n, int32_t row_ints, int32_t col0,
                 const int32_t* min_xyz, int64_t* codes, void* stream);

/* ------------------------------------------------------------------ convolution */

/* dst[r, :] = src[idx[r], :]  (rows of `channels` elements; src has num_src rows).  An idx
 * outside [0, num_src) yields a zero row and WCN_ERR_BOUNDS in dev_status (NULL: not reported).
 * Replaces the `comp_in_feats[in_map]` gather of _explicit_gemm_forward_logic
 * (warpconvnet/nn/functional/sparse_conv.py:309). */
int wcn_gather_rows(const void* src, int64_t num_src, const int32_t* idx, void* dst, int64_t num_rows,
                    int32_t channels, int dtype, int32_t* dev_status, void* stream);

/* dst[idx[r], :] += src[r, :]; idx must hold distinct rows (one kernel offset; dst has num_dst
 * rows).  An idx outside [0, num_dst) is skipped and reported like above.
 * Replaces `output_feature_tensor[out_map] += ...` (sparse_conv.py:310). */
int wcn_scatter_add_rows(const void* src, const int32_t* idx, void* dst, int64_t num_dst, int64_t num_rows,
                         int32_t channels, int dtype, int32_t* dev_status, void* stream);

/* Bytes of the packed-weight buffer wcn_conv_fwd needs for (algo, shape, dtype); 0 when
 * the chosen kernel reads the weights as given. */
int wcn_conv_packed_weight_bytes(int algo, int32_t num_offsets, int32_t c_in, int32_t c_out,
                                 int dtype, int64_t* bytes);

/* Re-layout weight[K, c_in, c_out] into the buffer above (K-major tiles for the tensor-core
 * kernel).  No reference counterpart (its kernels read the weights as stored). */
int wcn_conv_pack_weight(int algo, const void* weight, int32_t num_offsets, int32_t c_in,
                         int32_t c_out, int dtype, void* packed, void* stream);

/* Bytes of `workspace` wcn_conv_fwd needs for this problem on the current device (0: none).  Only
 * the tensor-core kernel uses one, when it divides the kernel offsets of a row block among several
 * CTAs (see split_k below): S * num_out * c_out fp32 partial sums.
 * Replaces the cudaMalloc inside the reference's split-K launcher
 * (warpconvnet/csrc/implicit_gemm_split_k.cu:254-258). */
int wcn_conv_workspace_bytes(int algo, int64_t num_out, int32_t num_offsets, int32_t c_in, int32_t c_out,
                             int dtype, int out_dtype, int32_t split_k, int64_t* bytes);

/* Output-stationary sparse convolution with a fused epilogue:
 *   acc[s, :] = sum_k feats[nbr[k*M + s], :] @ weight[k]      (rows with nbr < 0 skipped, fp32 accumulation)
 *   m = out_rows[s]           (out_rows NULL: m = s; else a permutation of 0..M-1, see
 *                              wcn_kmap_tile_order, with nbr being that call's nbr_tiled)
 *   y = acc * scale + shift   (scale NULL: y = acc + shift; both NULL: y = acc)
 *   y += residual[m, :]       (residual NULL: skipped; residual has the output dtype)
 *   y = max(y, 0)             (relu != 0)
 *   out[m, :] = (out dtype) y
 * feats / weight share `dtype`; scale / shift are fp32 [c_out].  Each output row is written
 * once by the block that owns it: no atomics, bit-reproducible.
 * feats_ld / residual_ld / out_ld are the distances between consecutive rows of the three
 * matrices in elements (0 = dense: c_in / c_out), so a matrix may be a column block of a wider
 * one (a skip connection's half of a concatenated buffer); rows must start on 16-byte boundaries
 * for the tensor-core kernel.  nbr entries >= num_in count as absent and raise WCN_ERR_BOUNDS.
 * num_in and M are below 2^31 (row numbers are 32-bit); larger values return WCN_ERR_INVALID_PARAMETERS.
 * algo WCN_CONV_TCGEN05 needs dtype f16/bf16, c_in % 32 == 0, c_out % 16 == 0, 16 <= c_out <= 256
 * and `packed_weight` from wcn_conv_pack_weight; WCN_CONV_AUTO picks it when those hold and
 * packed_weight is not NULL, else the SIMT kernel.
 * split_k: the tensor-core kernel may divide the kernel offsets of a 128-row block among S CTAs
 * (slice s owns offsets [s*K/S, (s+1)*K/S)), each leaving fp32 partial sums in `workspace`, which
 * a second kernel adds in slice order before the epilogue: for problems with fewer row blocks
 * than multiprocessors.  0 = the library decides, 1 = never, 2..16 = that many slices; a negative
 * value divides the OUTPUT COLUMNS into -split_k blocks instead (a tuning aid).  `workspace` must
 * hold wcn_conv_workspace_bytes(...) for the same arguments (NULL / 0 when that is 0).  Results
 * are the same bits on every run for a given S; different S round differently (fp32 sums are
 * grouped by slice).
 * Replaces implicit_gemm (warpconvnet/csrc/warpconvnet_pybind.cpp:732-837,
 * warpconvnet/csrc/implicit_gemm.cu:44-267) and cutlass_gemm_AD_gather_scatter with its
 * split_k_slices argument (warpconvnet_pybind.cpp:396-509,
 * warpconvnet/csrc/cutlass_gemm_gather_scatter.cu:176-464), the per-offset loop around them
 * (warpconvnet/nn/functional/sparse_conv.py:396-413, 516-544), the bias add
 * (sparse_conv.py:1794-1795) and the BatchNorm1d / ReLU / residual-add / concatenation chain of
 * the model blocks (examples/mink_unet.py:36-47, 129-141, 340-358). */
int wcn_conv_fwd(int algo, const void* feats, int64_t num_in, int64_t feats_ld, const void* weight,
                 const void* packed_weight, const int32_t* nbr, const int32_t* out_rows, int64_t num_out,
                 int32_t num_offsets, int32_t c_in, int32_t c_out, int dtype, const float* scale,
                 const float* shift, const void* residual, int64_t residual_ld, int relu, void* out,
                 int64_t out_ld, int out_dtype, int32_t split_k, void* workspace, int64_t workspace_bytes,
                 int32_t* dev_status, void* stream);

/* Pooling over a kernel map: out[m, :] = op over the offsets k with nbr[k*M + m] >= 0 of
 * feats[nbr[k*M + m], :] (fp32 accumulation, offsets in ascending order; rows without a neighbour
 * become 0; mean divides by the number of neighbours).  With the transposed table of a
 * non-overlapping pooling it is the un-pooling gather.  nbr entries >= num_in count as absent
 * and raise WCN_ERR_BOUNDS in dev_status (NULL: not reported).
 * Replaces kernel_map.to_csr() + row_reduction / torch_scatter.segment_csr of sparse_reduce
 * (warpconvnet/nn/functional/sparse_pool.py:87-92, warpconvnet/ops/reductions.py:36-70) and the
 * argsort + gather of sparse_unpool (sparse_pool.py:168-172). */
int wcn_row_reduce(const void* feats, int64_t num_in, const int32_t* nbr, int64_t num_out, int32_t num_offsets,
                   int32_t channels, int dtype, int op, void* out, int32_t* dev_status, void* stream);

/* Convolution in which every output row has exactly one (input row, kernel offset) pair, run from the
 * INPUT side on the tensor cores: a 1x1x1 convolution (optionally writing through a row permutation)
 * and a transposed convolution whose window equals its stride (2x2x2, stride 2).  For input row j and
 * offset k, out[dst_rows[k * num_in + j], :] = epilogue(feats[j, :] @ weight[k]); entries < 0 name no
 * output row.  dst_rows == NULL (num_offsets must be 1) means dst = j.  The caller guarantees that no
 * output row is named twice (it would be written twice, last writer wins) — for the stride-2 case
 * dst_rows is the [8, num_coarse] neighbour table of the matching strided convolution.
 * Feature rows arrive through TMA tiles (16-byte aligned base and pitch), weights (packed by
 * wcn_conv_pack_weight at width c_out_packed, a multiple of 16 >= c_out whose extra columns are zero)
 * stay in shared memory; fp16 / bf16 features, c_in % 32 == 0, c_out_packed <= 256.
 * The reference runs these layers through the same gather-GEMM-scatter as every other convolution
 * (warpconvnet/nn/functional/sparse_conv.py:358-415 with the swapped kernel map of :1916-1945). */
int wcn_conv_rows_supported(int32_t num_offsets, int32_t c_in, int32_t c_out_packed, int dtype, int out_dtype,
                            int32_t* supported);
int wcn_conv_rows_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed_weight,
                      const int32_t* dst_rows, int64_t num_out, int32_t num_offsets, int32_t c_in,
                      int32_t c_out_packed, int32_t c_out, int dtype, const float* scale, const float* shift,
                      const void* residual, int64_t residual_ld, int relu, void* out, int64_t out_ld,
                      int out_dtype, int32_t* dev_status, void* stream);

/* Weight gradient of the convolution above, accumulated into grad_weight[K, c_in, c_out] (fp32; the
 * caller zeroes it):
 *   grad_weight[k] += feats[nbr[k*M + m], :]^T (outer) grad_out[m, :]   over rows m with nbr >= 0
 * feats / grad_out share `dtype` (f16 or bf16), fp32 accumulation on the tensor cores; the partial
 * sums of different row ranges are added with atomics, so the last bits vary from run to run.
 * Needs c_in % 32 == 0, c_out % 32 == 0, c_out <= 256; else WCN_ERR_UNSUPPORTED_CONFIG (callers fall
 * back to a GEMM per offset).  (`nbr`, `out_rows`) is the pair wcn_conv_fwd takes: the plain table
 * with out_rows NULL, or the tiled one with its row order (grad_out is then read at out_rows[s]);
 * `tile_masks` (from wcn_kmap_tile_masks on the same table, or NULL) lets the kernel skip the 128-row
 * steps in which the offsets of a CTA have no neighbour.
 * Replaces cutlass_gemm_trAB_gather (warpconvnet/csrc/warpconvnet_pybind.cpp:511-624) and
 * split_k_implicit_gemm (warpconvnet/csrc/implicit_gemm_split_k.cu:63-393) with the per-offset loop
 * around them (warpconvnet/nn/functional/sparse_conv.py:591-604). */
int wcn_conv_wgrad(const void* feats, int64_t num_in, const void* grad_out, const int32_t* nbr,
                   const int32_t* out_rows, const uint32_t* tile_masks, int64_t num_out, int32_t num_offsets, int32_t c_in, int32_t c_out, int dtype,
                   float* grad_weight, int32_t* dev_status, void* stream);

/* ------------------------------------------------------------------ self test */

/* Checks the library's bounded device-side waits: launches one small kernel that waits, with a
 * limit of `limit_cycles` SM clock cycles (1e3 .. 2e9), for a barrier phase that nothing can
 * complete.  The wait must give up, store WCN_ERR_WAIT_EXPIRED in dev_status and let the kernel
 * end normally; gave_up (device int32, may be NULL) receives 1 when it did.  The context stays
 * usable.  No counterpart in the reference (its kernels have no device-side waits). */
int wcn_selftest_bounded_wait(int64_t limit_cycles, int32_t* dev_status, int32_t* gave_up, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WCN_B200_H_ */
