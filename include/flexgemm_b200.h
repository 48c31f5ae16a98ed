/*
 * flexgemm_b200 -- C ABI of the sm_100a submanifold-conv3d backend.
 *
 * Every function takes plain integers and device pointers and launches on the
 * given CUDA stream (pass the cudaStream_t as a void*).  The library allocates
 * nothing: outputs, tables and workspaces are owned by the caller (the entry
 * points whose name ends in _bytes tell how much to provide).  Nothing
 * synchronises the stream.
 *
 * Return value: 0 on success, a negative FGB_E_* code when the arguments are
 * rejected before any launch, or 1000 + cudaError_t when a launch failed.
 * Soft errors detected on the device (a hash probe or a barrier wait that ran
 * out of iterations) do not trap: the kernel records a non-zero code in the
 * caller's `status` word (int32 in device memory, zeroed by the caller) and
 * finishes; read it at the next synchronisation point.
 *
 * The citations name the interface of FlexGEMM (paths inside its source tree)
 * that each entry point stands in for.
 */
#ifndef FLEXGEMM_B200_H_
#define FLEXGEMM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FGB_OK 0
#define FGB_E_NULL (-1)       /* a required pointer is null            */
#define FGB_E_SIZE (-2)       /* a size or count is out of range       */
#define FGB_E_DTYPE (-3)      /* unsupported dtype / key width         */
#define FGB_E_ALIGN (-4)      /* pointer or channel count misaligned   */
#define FGB_E_WORKSPACE (-5)  /* workspace too small                   */
#define FGB_E_DRIVER (-6)     /* CUDA driver entry point unavailable   */
#define FGB_E_STATIC_LIMIT (-7) /* larger than a no-allocation entry point's built-in scratch */
#define FGB_E_CUDA_BASE 1000  /* 1000 + cudaError_t                    */

/* device-side status codes (written to *status) */
#define FGB_S_TABLE_FULL 1    /* hash insert found no free slot        */
#define FGB_S_WAIT_TIMEOUT 2  /* a bounded barrier wait ran out        */

/* element types of features / weights */
#define FGB_F16 0
#define FGB_BF16 1
#define FGB_F32_TF32 2  /* fp32 storage, TF32 tensor-core math (allow_tf32 = True)  */
#define FGB_F32_IEEE 3  /* fp32 storage, fp32-accurate math   (allow_tf32 = False) */

/* activation of the fused forward epilogue */
#define FGB_ACT_NONE 0
#define FGB_ACT_SILU 1  /* x * sigmoid(x) */

const char* fgb_version(void);
const char* fgb_error_string(int code);

/* Host-only self-test of the per-device caches the launch code keeps (SM count,
 * dynamic shared-memory limit per kernel and device); touches no GPU.  Returns 0
 * or the number of the failed expectation.  (No counterpart in the reference.) */
int fgb_selftest_device_tables(void);

/* cudaMemcpyAsync(host_dst, device_src, bytes, device-to-host) on `stream`: how
 * a caller fetches valid_signal_seg[V] (the pair count) and its status word
 * after fgb_subm_build_neighbor_map without leaving the stream.  host_dst
 * should be pinned. */
int fgb_fetch_words_async(void* host_dst, const void* device_src, int64_t bytes, void* stream);

/* ------------------------------------------------------------------------
 * Hash table + neighbour map
 * --------------------------------------------------------------------- */

/* Bytes of table storage for `slots` slots.  key_bits is 32 when
 * B*W*H*D < 2^32 and 64 otherwise -- the same rule as init_hashmap
 * (flex_gemm/ops/utils.py:4-19).  Returns a negative code on bad arguments. */
int64_t fgb_hash_table_bytes(int64_t slots, int key_bits);

/* Number of 256-voxel blocks the map kernels use for `n` voxels (sizes the
 * block_offsets array below). */
int64_t fgb_map_num_blocks(int64_t n);

/* Builds the table from `coords` and fills the [n, V] neighbour map,
 * V = Kw*Kh*Kd: neighbor_map[i, v] is the row of the voxel at
 * coords[i] + (k - K/2) * dilation for v = (kx*Kh + ky)*Kd + kz, or
 * 0xffffffff.  Also writes the per-voxel validity mask gray_code[i] (bit v set
 * iff valid), its Gray-to-binary decode binary_code[i], block_offsets
 * [V * nblk] (for offset v and 256-voxel block k, the number of valid pairs of
 * offset v in the blocks before k) and valid_signal_seg[V + 2]: V + 1 entries
 * of the exclusive prefix of the per-offset totals (entry V is the pair count
 * L), followed by one word that is 0 when the rows were found in key order (the
 * table-free path built the map) and non-zero otherwise; fgb_pp_valid_signal
 * takes a pointer to that word.
 *
 * Stands in for hashmap_build_submanifold_conv_neighbour_map
 * (flex_gemm/kernels/cuda/spconv/subm_neighbor_map.cu:104-162, with
 * hashmap_insert_3d_idx_as_val, kernels/cuda/hash/hash.cu:369-449) and for the
 * gray/binary pass of neighbor_map_post_process_for_masked_implicit_gemm_1
 * (kernels/cuda/spconv/migemm_neighmap_pp.cu:19-44, 85-154).
 *
 * coords: int32 [n,4] (b,x,y,z), 16-byte aligned.  table: fgb_hash_table_bytes
 * bytes; its content on entry is ignored.  slots >= n.  V <= 32.
 *
 * Rows that arrive in ascending flat-index order -- lexicographic (b, x, y, z),
 * without duplicates, batch indices below B -- need no hash table (a row's
 * position is its rank among the keys, and a (b, x, y) column is a run of
 * consecutive rows): a kernel checks the order on the device, without a host
 * round trip, and records where every column starts and ends in a direct-address
 * table of B*W*H entries of 8 bytes kept in `table`; the lookup then reads the
 * neighbouring column's entry and searches its few rows.  This path is taken
 * when B*W*H*8 <= fgb_hash_table_bytes(slots, key_bits); otherwise, and for
 * unsorted rows, the hash table is built and probed.  The map is the same either
 * way.  B = number of samples (coords[:,0] < B); B = 0 disables the table-free
 * path. */
int fgb_subm_build_neighbor_map(const int32_t* coords, int64_t n,
                                int B, int W, int H, int D,
                                int Kw, int Kh, int Kd,
                                int Dw, int Dh, int Dd,
                                void* table, int64_t slots, int key_bits,
                                uint32_t* neighbor_map,
                                int32_t* gray_code, int32_t* binary_code,
                                uint32_t* block_offsets, uint32_t* valid_signal_seg,
                                int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * Post-processing for the masked implicit GEMM
 * --------------------------------------------------------------------- */

/* Workspace bytes for fgb_pp_sorted_idx. */
int64_t fgb_pp_sorted_idx_workspace_bytes(int64_t n);

/* sorted_idx (int64 [n]) = the stable argsort of binary_code (signed int32,
 * only bits [0, key_bits) differ): a radix sort with 9-bit digits, one kernel
 * per digit (three for a 3x3x3 stencil), the tiles of a pass chained by a
 * decoupled look-back.  n < 2^30.  A look-back that stays unanswered (it never
 * should) records FGB_S_WAIT_TIMEOUT in *status (may be null) instead of
 * spinning.  Stands in for torch::argsort(binary_code) in
 * migemm_neighmap_pp.cu:79, 221 (an unstable sort there; any order of equal
 * codes is a valid result, this one is the stable one and hence deterministic). */
int fgb_pp_sorted_idx(const int32_t* binary_code, int64_t n, int key_bits,
                      int64_t* sorted_idx, void* workspace, int64_t workspace_bytes,
                      int32_t* status, void* stream);

/* Pair lists for wgrad: grouped by offset v, ascending output row inside a
 * group: valid_signal_o[p] = row, valid_signal_i[p] = neighbor_map[row, v].
 * `block_offsets` and `valid_signal_seg` are the arrays written by
 * fgb_subm_build_neighbor_map.  The lists need valid_signal_seg[V] entries.
 * unsorted_flag (device, may be null): &valid_signal_seg[V + 1] of a
 * submanifold build.  When it holds 0 the rows are in key order; a translation
 * keeps that order, so valid_signal_i of offset v equals valid_signal_o of the
 * opposite offset V-1-v and both lists are written from the masks alone,
 * without reading the map.  Null (the generic strided conv, whose map has no
 * such symmetry) or non-zero: the lists are gathered from the map.
 * Stands in for the cumsum + gather_idx_val_seg_from_prefix_sum_kernel part of
 * neighbor_map_post_process_for_masked_implicit_gemm_1
 * (migemm_neighmap_pp.cu:157-178, 224-240). */
int fgb_pp_valid_signal(const uint32_t* neighbor_map, const int32_t* gray_code,
                        int64_t n, int V,
                        const uint32_t* block_offsets, const uint32_t* valid_signal_seg,
                        uint32_t* valid_signal_i, uint32_t* valid_signal_o,
                        const uint32_t* unsorted_flag, void* stream);

/* tile_masks[t] = OR of gray_code[sorted_idx[r]] over the rows r of tile t
 * (tile = `block` consecutive sorted rows, a power of two in [8, 1024]).
 * This is reduced_code of reduce_code_kernel (migemm_neighmap_pp.cu:246-296);
 * the conv kernels below consume it directly. */
int fgb_pp_tile_masks(const int32_t* gray_code, const int64_t* sorted_idx, int64_t n,
                      int block, uint32_t* tile_masks, void* stream);

/* Expands tile masks to the reference's list form:
 * valid_kernel_seg (int32 [nblk+1]) = exclusive prefix of popcounts,
 * valid_kernel (int32, capacity nblk*32) = ascending set-bit positions.
 * Stands in for neighbor_map_post_process_for_masked_implicit_gemm_2
 * (migemm_neighmap_pp.cu:299-368).  Single pass, one CTA; nblk <= 2^24. */
int fgb_pp_valid_kernel(const uint32_t* tile_masks, int64_t nblk,
                        int32_t* valid_kernel, int32_t* valid_kernel_seg, void* stream);

/* ------------------------------------------------------------------------
 * Masked implicit GEMM: fprop, dgrad, wgrad  (tcgen05 / TMEM, tile M = 128)
 * --------------------------------------------------------------------- */

/* Rows per tile used by the conv kernels: tile_masks passed to them must have
 * been built with block == fgb_conv_tile_rows(). */
int fgb_conv_tile_rows(void);

/* Caps the number of CTAs (one per SM) that the persistent fprop / dgrad kernels
 * launch from now on; 0 lifts the cap.  Returns the previous value.  For callers
 * that run a collective beside a conv kernel (the multi-GPU backward launches
 * its all-reduce before dgrad): the conv CTAs fill their SMs, so without a few
 * SMs left over the collective's kernel would only start when the conv ends.
 * Process-wide; read when a kernel is launched. */
int fgb_conv_set_cta_limit(int max_ctas);

/* Split-K of fprop / dgrad.  A launch with fewer work items (256-row blocks x
 * column tiles) than half the SMs cuts every item into shares of its offsets that
 * run as separate items into fp32 slabs in the workspace; a second kernel adds
 * the slabs in a fixed order, adds the bias and converts (deterministic).  This
 * setting overrides the rule: 0 = automatic (as many shares as SMs per item, at
 * most V), 1 = never split, k = k shares.  Returns the previous value.
 * Process-wide; read when workspace sizes are computed and when a kernel is
 * launched, so change it between calls, not between the size query and the call.
 * Stands in for the SPLITK heuristic of the reference's kernels
 * (sparse_submanifold_conv_fwd_masked_implicit_gemm_splitk.py:109-121). */
int fgb_conv_set_splitk(int splits);

/* dgrad of 16-bit types reads the weight as it is stored ([Co][V][Ci]) as an
 * MN-major tensor-core operand; 32-bit types and column tiles under 64 channels
 * work on a re-laid-out copy ([Ci][V][Co]) made by a kernel of the call.  on = 1
 * forces the copy for every type (0 = default); returns the previous setting.
 * The results are the same bit for bit.  Process-wide; read at launch. */
int fgb_conv_set_dgrad_relayout(int on);

/* block_order (uint32 [ceil(num_tiles / 2)]) = the 256-row blocks (pairs of
 * consecutive 128-row tiles) in descending order of work, computed from the tile
 * masks.  The persistent conv kernels deal blocks to the SMs from this list so
 * that every SM gets about the same amount of work; passing a null block_order
 * to them means natural order.  (The reference balances by launching one CTA
 * per tile; it has no counterpart of this list.) */
int fgb_conv_block_schedule(const uint32_t* tile_masks, int64_t num_tiles,
                            uint32_t* block_order, void* stream);

/* out[r, :] = bias + sum_v feats[neighbor_map[r, v], :] * weight[:, v, :]^T
 * for every row r, visiting only the offsets set in the row's tile mask.
 * feats [n, Ci], weight [Co, V, Ci], bias [Co] or null, out [n, Co]; all of
 * element type `dtype`, rows 16-byte aligned (Ci, Co multiples of 8 for 16-bit
 * types, of 4 for fp32).  tile_masks: fgb_pp_tile_masks with block = 128.
 * Stands in for sparse_submanifold_conv_fwd_masked_implicit_gemm_splitk
 * (flex_gemm/kernels/triton/spconv/
 *  sparse_submanifold_conv_fwd_masked_implicit_gemm_splitk.py:21-172).
 * `workspace`: fgb_conv_workspace_bytes(0, ...) bytes, 256-byte aligned (it holds
 * the work counter of the persistent kernel, the split operands for
 * FGB_F32_IEEE, and the fp32 slabs of a split-K launch, see
 * fgb_conv_set_splitk). */
int fgb_subm_conv_fprop(const void* feats, const void* weight, const void* bias,
                        const uint32_t* neighbor_map, const int64_t* sorted_idx,
                        const uint32_t* tile_masks, const uint32_t* block_order,
                        void* out, int64_t n, int Ci, int Co, int V, int dtype,
                        void* workspace, int64_t workspace_bytes,
                        int32_t* status, void* stream);

/* fgb_subm_conv_fprop with the elementwise work that follows a conv in a residual
 * block done in its epilogue:
 *   y = conv(feats) + bias                 rounded to `dtype`
 *   preact_out[r, :] = y                   when preact_out is not null (what the
 *                                          backward of the activation needs)
 *   out[r, :] = activation(y) + residual[r, :]
 * activation: FGB_ACT_NONE or FGB_ACT_SILU, computed in fp32; residual [n, Co] of
 * `dtype`, 16-byte aligned, or null.  With an activation and a residual the
 * activation's result is rounded to `dtype` before the add, so the result has
 * the roundings of the unfused sequence conv -> activation -> add.  The
 * reference has no such call: its callers run torch elementwise kernels between
 * convs (the residual stack [conv, SiLU, conv] + skip). */
int fgb_subm_conv_fprop_fused(const void* feats, const void* weight, const void* bias,
                              const void* residual,
                              const uint32_t* neighbor_map, const int64_t* sorted_idx,
                              const uint32_t* tile_masks, const uint32_t* block_order,
                              void* out, void* preact_out,
                              int64_t n, int Ci, int Co, int V, int dtype, int activation,
                              void* workspace, int64_t workspace_bytes,
                              int32_t* status, void* stream);

/* grad_feats[r, :] = sum_v grad_out[neighbor_map[r, v], :] * weight[:, V-1-v, :]
 * grad_out [n, Co], weight [Co, V, Ci], grad_feats [n, Ci].  The workspace
 * holds the re-laid-out weight [Ci, V, Co] (fgb_conv_workspace_bytes).
 * Stands in for sparse_submanifold_conv_bwd_input_masked_implicit_gemm_splitk
 * (…/sparse_submanifold_conv_bwd_masked_implicit_gemm_splitk.py:23-100, 205-251). */
int fgb_subm_conv_dgrad(const void* grad_out, const void* weight,
                        const uint32_t* neighbor_map, const int64_t* sorted_idx,
                        const uint32_t* tile_masks, const uint32_t* block_order,
                        void* grad_feats, int64_t n, int Ci, int Co, int V, int dtype,
                        void* workspace, int64_t workspace_bytes,
                        int32_t* status, void* stream);

/* Workspace bytes for fprop (pass = 0), dgrad (pass = 1) and wgrad (pass = 2,
 * with the given split count) on n rows.  FGB_F32_IEEE needs room for the
 * hi/lo-split copies of its operands, hence the dependence on n. */
int64_t fgb_conv_workspace_bytes(int pass, int64_t n, int Ci, int Co, int V, int dtype, int splitk);

/* Split count the library would pick for wgrad on the current device (room for one wave of units). */
int fgb_wgrad_default_splitk(int64_t n_pairs, int Ci, int Co, int V, int dtype);

/* grad_weight[co, v, ci] = sum_{p in segment v} grad_out[valid_signal_o[p], co]
 *                                              * feats[valid_signal_i[p], ci]
 * The pair lists are cut into units of equal length (an offset with more pairs
 * gets more units).  `splitk` is the budget: the workspace holds (splitk + 1) * V
 * partials, and the kernel uses the largest whole number of waves of CTAs (one
 * per SM) that fits it, planning the unit length from valid_signal_seg on the
 * device.  Each unit's fp32 partial [Co, Ci] goes to the workspace and the
 * partials of an offset are then added in a fixed order (deterministic).  n_pairs is the length of the pair
 * lists (valid_signal_seg[V]).  grad_weight (element type `dtype`) and/or
 * grad_weight_f32 may be null; the fp32 copy is what a multi-GPU caller hands
 * to its all-reduce.
 * block_offsets (may be null): the [V, nblk] array written by
 * fgb_subm_build_neighbor_map.  With it the lists of all offsets are cut at the
 * same output rows into row bands, and every CTA walks its share of band after
 * band, so that the whole launch reads one band of rows of grad_out and feats at
 * a time and the 27 offsets share it in L2 instead of each streaming both
 * matrices from HBM; without it every CTA walks one contiguous piece of one
 * list.  The result does not depend on it beyond the order of fp32 additions.
 * Stands in for sparse_submanifold_conv_bwd_weight_masked_implicit_gemm_splitk
 * (…/sparse_submanifold_conv_bwd_masked_implicit_gemm_splitk.py:107-182, 274-317). */
int fgb_subm_conv_wgrad(const void* grad_out, const void* feats,
                        const uint32_t* valid_signal_i, const uint32_t* valid_signal_o,
                        const uint32_t* valid_signal_seg, const uint32_t* block_offsets,
                        void* grad_weight, float* grad_weight_f32,
                        int64_t n, int64_t n_pairs, int Ci, int Co, int V, int dtype, int splitk,
                        void* workspace, int64_t workspace_bytes,
                        int32_t* status, void* stream);

/* Number of row bands fgb_*_conv_wgrad cuts the pair lists into when it is given
 * block_offsets: 0 = chosen from the sizes (one band while grad_out and feats fit
 * the L2 together, bands of about 8 MB of rows beyond that), 1 .. 64 = fixed.  Returns the previous value.  Process-wide tuning knob; read at launch. */
int fgb_wgrad_set_row_bands(int bands);

/* Host-side replay of how a wgrad launch splits the pair lists among its CTAs, for
 * tests (no GPU involved; seg and block_offsets are HOST arrays here, block_offsets
 * may be null).  For unit u (offset-major) and band b,
 * plan[(u * bands + b) * 3 + 0 / 1 / 2] = first pair / number of k-blocks / end of
 * the band in the pair list; a k-block is *kb_out consecutive pairs, cut at the
 * band's end.  Returns the number of units or a negative code.  (No counterpart in
 * the reference.) */
int fgb_wgrad_plan_host(const uint32_t* seg, const uint32_t* block_offsets, int64_t n_out, int64_t n_in,
                        int Ci, int Co, int V, int dtype, int splitk,
                        uint32_t* plan, int64_t plan_capacity, int* bands_out, int* kb_out);

/* grad_bias[c] = sum_r grad_out[r, c] accumulated in fp32; writes grad_bias
 * (element type `dtype`) and/or grad_bias_f32, either may be null.
 * Stands in for grad_output.sum(0)
 * (…/sparse_submanifold_conv_bwd_masked_implicit_gemm_splitk.py:365-366).
 * workspace: fgb_bias_grad_workspace_bytes(Co). */
int64_t fgb_bias_grad_workspace_bytes(int Co);
int fgb_subm_conv_bias_grad(const void* grad_out, void* grad_bias, float* grad_bias_f32,
                            int64_t n, int Co, int dtype,
                            void* workspace, int64_t workspace_bytes, void* stream);

/* Bias gradient for callers that cannot allocate device memory.
 * (No counterpart in the reference: its bias gradient is a torch reduction that
 * allocates freely.)
 *
 * Same result as fgb_subm_conv_bias_grad, but the caller passes no workspace:
 * the fp32 partial sums live in a fixed buffer inside the library image
 * (592 * 2048 floats = 4.6 MiB, resident on every GPU that loads the library,
 * for the life of the process).  Meant for hosts that give a plug-in a fixed
 * arena and forbid cudaMalloc, and for loops that cannot tolerate the
 * device-wide synchronisation an allocation implies.  The call itself performs
 * no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 *  - Co must be <= fgb_noalloc_max_channels() (2048); larger returns
 *    FGB_E_STATIC_LIMIT and launches nothing.
 *  - The first call on each device looks up the buffer's device address
 *    (cudaGetSymbolAddress, with that device current).  Make that first call
 *    before starting any stream capture.
 *  - All calls on a device share the one buffer, and it keeps whatever the last
 *    call left in it.  Nothing needs clearing (each call overwrites every value
 *    it later reads), but two calls that overlap on the GPU -- different
 *    streams without an ordering between them -- race on it.  Serialise them. */
int fgb_noalloc_max_channels(void);
int fgb_subm_conv_bias_grad_noalloc(const void* grad_out, void* grad_bias, float* grad_bias_f32,
                                    int64_t n, int Co, int dtype, void* stream);

/* dst (element type `dtype`) = src (fp32), count elements: the cast applied to
 * an all-reduced fp32 gradient. */
int fgb_cast_from_f32(const float* src, void* dst, int64_t count, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Generic sparse convolution (stride / padding / dilation, output voxels that
 * differ from the input voxels): the caller on either side of a submanifold
 * conv in a network (down- and up-sampling).  Same hash table, sort,
 * pair-list and GEMM kernels; separate forward and backward maps.
 * Reference: flex_gemm/ops/spconv/sparse_conv3d.py:59-539,
 * flex_gemm/kernels/cuda/spconv/sparse_neighbor_map.cu.
 * --------------------------------------------------------------------- */

/* Output grid extents: Wo = (W + 2*Pw - Dw*(Kw-1) - 1) / Sw + 1, etc.
 * (sparse_neighbor_map.cu:89-91). */
int fgb_sparse_out_grid(int W, int H, int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd,
                        int Pw, int Ph, int Pd, int Dw, int Dh, int Dd, int* Wo, int* Ho, int* Do);

/* Output coordinates, step 1 of 2.  Every input voxel proposes, for every
 * kernel offset k, the output voxel (c + P - k*Dil) / S when that is integral
 * and inside the output grid; a hash set (`set`: `slots` words of key_bits
 * bits, any contents) removes duplicates and `keys` (capacity `slots` words of
 * key_bits bits) receives the flat (b, x, y, z) index of each distinct output
 * voxel in arbitrary order; *count (device) = how many.  key_bits is 32 when
 * B*Wo*Ho*Do < 2^32 - 1, else 64.  A set that fills up records
 * FGB_S_TABLE_FULL.  Stands in for the insert half of
 * hashmap_build_sparse_conv_out_coords (sparse_neighbor_map.cu:18-56, 103-124). */
int fgb_sparse_out_coords_collect(const int32_t* in_coords, int64_t n_in, int W, int H, int D,
                                  int Kw, int Kh, int Kd, int Sw, int Sh, int Sd,
                                  int Pw, int Ph, int Pd, int Dw, int Dh, int Dd,
                                  void* set, int64_t slots, int key_bits,
                                  void* keys, uint32_t* count, int32_t* status, void* stream);

/* Output coordinates, step 2 of 2 (after the caller has read *count): sorts
 * the keys by serialisation key and decodes them to out_coords (int32
 * [count, 4], rows (b, x, y, z)).  mode 0 = flat bxyz index, 1 = Morton code,
 * 2 = Hilbert index; for modes 1 and 2 coord_bits is the bit length of
 * max(W, H, D) - 1 and the batch index sits above 3*coord_bits bits
 * (sparse_neighbor_map.cu:126-196, utils.h:24-106).  B = batch size. */
int64_t fgb_sparse_out_coords_workspace_bytes(int64_t count, int key_bits, int mode);
int fgb_sparse_out_coords_finalize(const void* keys, int64_t count, int key_bits, int mode, int coord_bits,
                                   int B, int W, int H, int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd,
                                   int Pw, int Ph, int Pd, int Dw, int Dh, int Dd,
                                   void* workspace, int64_t workspace_bytes, int32_t* out_coords, void* stream);

/* Forward map neighbor_map[o, v] = row of the input voxel at
 * out_coords[o] * S - P + k * Dil (v = (kx*Kh + ky)*Kd + kz) or 0xffffffff, and
 * -- when neighbor_map_bwd is non-null -- the backward map
 * neighbor_map_bwd[i, v] = o for every hit (other entries 0xffffffff).  The
 * table (fgb_hash_table_bytes(slots, key_bits) bytes, slots >= n_in) is built
 * over the input voxels.  gray_code / binary_code / block_counts /
 * valid_signal_seg describe the FORWARD map as in
 * fgb_subm_build_neighbor_map (block_counts sized by fgb_map_num_blocks(n_out);
 * valid_signal_seg has V + 1 entries here: there is no key-order word, pass a
 * null unsorted_flag to fgb_pp_valid_signal).
 * Stands in for hashmap_build_sparse_conv_neighbour_map
 * (sparse_neighbor_map.cu:405-568). */
int fgb_sparse_build_neighbor_map(const int32_t* in_coords, int64_t n_in,
                                  const int32_t* out_coords, int64_t n_out,
                                  int W, int H, int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd,
                                  int Pw, int Ph, int Pd, int Dw, int Dh, int Dd,
                                  void* table, int64_t slots, int key_bits,
                                  uint32_t* neighbor_map, uint32_t* neighbor_map_bwd,
                                  int32_t* gray_code, int32_t* binary_code,
                                  uint32_t* block_counts, uint32_t* valid_signal_seg,
                                  int32_t* status, void* stream);

/* gray_code / binary_code of an existing map (used for the backward map, whose
 * entries are scattered and therefore cannot be summarised while it is built).
 * Stands in for the mask half of ..._1_no_bwd (migemm_neighmap_pp.cu:58-82). */
int fgb_pp_gray_code(const uint32_t* neighbor_map, int64_t n, int V,
                     int32_t* gray_code, int32_t* binary_code, void* stream);

/* The conv passes with distinct input and output row counts.  fprop: the map
 * has n_out rows and feats n_in rows.  dgrad: the BACKWARD map has n_in rows,
 * grad_out n_out rows, and offset v uses weight slot v (no mirroring).  wgrad:
 * pair lists from the forward map.  Workspaces are sized by
 * fgb_sparse_conv_workspace_bytes (pass 0/1/2 as in fgb_conv_workspace_bytes). */
int fgb_sparse_conv_fprop(const void* feats, const void* weight, const void* bias,
                          const uint32_t* neighbor_map, const int64_t* sorted_idx,
                          const uint32_t* tile_masks, const uint32_t* block_order,
                          void* out, int64_t n_out, int64_t n_in, int Ci, int Co, int V, int dtype,
                          void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);
int fgb_sparse_conv_dgrad(const void* grad_out, const void* weight,
                          const uint32_t* neighbor_map_bwd, const int64_t* sorted_idx_bwd,
                          const uint32_t* tile_masks_bwd, const uint32_t* block_order_bwd,
                          void* grad_feats, int64_t n_in, int64_t n_out, int Ci, int Co, int V, int dtype,
                          void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);
int fgb_sparse_conv_wgrad(const void* grad_out, const void* feats,
                          const uint32_t* valid_signal_i, const uint32_t* valid_signal_o,
                          const uint32_t* valid_signal_seg, const uint32_t* block_offsets,
                          void* grad_weight, float* grad_weight_f32,
                          int64_t n_out, int64_t n_in, int64_t n_pairs, int Ci, int Co, int V, int dtype, int splitk,
                          void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);
int64_t fgb_sparse_conv_workspace_bytes(int pass, int64_t n_out, int64_t n_in, int Ci, int Co, int V, int dtype, int splitk);

/* ------------------------------------------------------------------------
 * Generic use of the coordinate table, and the sparse grid sample built on it
 * (flex_gemm/ops/grid_sample/grid_sample.py, kernels/cuda/grid_sample/
 * grid_sample.cu, kernels/cuda/hash/hash.cu, kernels/triton/grid_sample/).
 * --------------------------------------------------------------------- */

/* The library's own packed table (one 64-bit word per slot for 32-bit keys; the
 * layout the neighbour-map and grid-sample kernels probe): clears it and inserts
 * coords[i] -> i.  Plays the part of hashmap_insert_3d_idx_as_val
 * (hash/hash.cu:369-449) inside grid_sample_3d.  slots >= n. */
int fgb_hash_insert_3d_idx_as_val(const int32_t* coords, int64_t n, int W, int H, int D,
                                  void* table, int64_t slots, int key_bits, int32_t* status, void* stream);

/* out_rows[i] = row stored for query_coords[i] (int32 [m,4] rows (b,x,y,z)) or
 * 0xffffffff; coordinates outside the grid are reported as absent.  Stands in
 * for hashmap_lookup_3d (hash/hash.cu:296-365). */
int fgb_hash_lookup_3d(const int32_t* query_coords, int64_t m, int W, int H, int D,
                       void* table, int64_t slots, int key_bits, uint32_t* out_rows, void* stream);

/* The generic hash map with caller-chosen values, in the reference's layout:
 * hashmap_keys (uint32 or uint64 [slots], empty = all ones, initialised by the
 * caller as init_hashmap does, flex_gemm/ops/utils.py:4-19) and hashmap_vals
 * (uint32 or uint64 [slots]); key_bits / val_bits are 32 or 64.  A lookup
 * returns all ones (of the value type) for an absent key.  Which slot a key
 * occupies is not part of the contract.  Inserting duplicate keys in one call
 * keeps one of their values.  A full table records FGB_S_TABLE_FULL in *status
 * (may be null).
 *   fgb_hashmap_insert         keys [m] -> values [m]        (hash/hash.cu:13-92)
 *   fgb_hashmap_lookup         values of keys [m]             (hash/hash.cu:94-175)
 *   fgb_hashmap_insert_3d      key = flat (b, x, y, z) index of coords [m,4],
 *                              truncated to the key type       (hash/hash.cu:177-270)
 *   fgb_hashmap_lookup_3d      the same keying; coordinates outside
 *                              [0,W)x[0,H)x[0,D) are absent    (hash/hash.cu:272-365)
 *   fgb_hashmap_insert_3d_idx_as_val   value = row number      (hash/hash.cu:369-449)
 * coords must be 16-byte aligned. */
int fgb_hashmap_insert(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                       const void* keys, const void* values, int64_t m, int32_t* status, void* stream);
int fgb_hashmap_lookup(const void* hashmap_keys, const void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                       const void* keys, int64_t m, void* out_values, void* stream);
int fgb_hashmap_insert_3d(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                          const int32_t* coords, const void* values, int64_t m, int W, int H, int D,
                          int32_t* status, void* stream);
int fgb_hashmap_insert_3d_idx_as_val(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                                     const int32_t* coords, int64_t m, int W, int H, int D,
                                     int32_t* status, void* stream);
int fgb_hashmap_lookup_3d(const void* hashmap_keys, const void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                          const int32_t* coords, int64_t m, int W, int H, int D, void* out_values, void* stream);

/* Neighbour map of B*L float query points (x, y, z) in voxel units, batch b =
 * point / L, against a table built by fgb_hash_insert_3d_idx_as_val.
 * trilinear == 0: neighbor[q] = row of the voxel (int)x, (int)y, (int)z
 * (grid_sample.cu:26-55).  trilinear != 0: neighbor[q, 0..7] / weight[q, 0..7]
 * = rows and normalised trilinear weights of the eight voxels around the point,
 * corner k at floor(q - 0.5) + (k & 1, (k >> 1) & 1, (k >> 2) & 1)
 * (grid_sample.cu:149-194); absent corners get 0xffffffff and weight 0 (the
 * reference leaves row 0 there for corners 1..7; their weight is 0 either way). */
int fgb_grid_sample_neighbor_map(const float* query, int64_t B, int64_t L, int W, int H, int D,
                                 void* table, int64_t slots, int key_bits, int trilinear,
                                 uint32_t* neighbor, float* weight, void* stream);

/* out[m, :] = sum_k weight[m, k] * feats[indices[m, k], :] over the valid
 * entries (weight may be null: all ones).  feats [*, C], out [M, C] of element
 * type dtype, indices uint32 [M, V], weight fp32 [M, V]; C % 4 == 0.  Stands in
 * for indice_weighed_sum_fwd (kernels/triton/grid_sample/indice_weighed_sum_fwd.py). */
int fgb_indice_weighted_sum_fwd(const void* feats, const uint32_t* indices, const float* weight, void* out,
                                int64_t M, int C, int V, int dtype, void* stream);

/* grad_feats_f32[indices[m, k], :] += weight[m, k] * grad_out[m, :]; the fp32
 * buffer [N, C] is zeroed by the call and filled with atomic adds.  Stands in
 * for indice_weighed_sum_bwd_input (…/indice_weighed_sum_bwd.py), which adds
 * in the feature dtype. */
int fgb_indice_weighted_sum_bwd(const void* grad_out, const uint32_t* indices, const float* weight,
                                float* grad_feats_f32, int64_t M, int64_t N, int C, int V, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Pipeline microbenchmark (no counterpart in the reference)
 * --------------------------------------------------------------------- */

/* What one SM sustains of the traffic and the MMAs of an fprop / dgrad stage
 * (Ci = Co = 256, 16-bit), isolated from the conv kernel: per stage 32 KB of
 * rows gathered at random from rows[n_rows][row_bytes] (row_bytes a multiple
 * of 128), 32 KB of the dense operand from dense[dense_bytes] by TMA, and 8
 * MMAs 128 x 256 x 16 on whatever the stage buffers hold.  `mode` is a sum of
 *   FGB_MB_TMA      the dense-operand stream
 *   FGB_MB_GATHER   the gathered stream (cp.async, 16 bytes per thread)
 *   FGB_MB_MMA      the MMA stream
 *   FGB_MB_COUPLED  MMAs wait for full stages and free them by tcgen05.commit,
 *                   as in the conv kernel (else every stream runs by itself)
 *   FGB_MB_GATHER4  gather by TMA tile::gather4 instead of cp.async
 *   FGB_MB_PAIR     CTA pairs (tcgen05 cta_group::2, M = 256 over both CTAs,
 *                   16 KB of the dense operand per CTA); implies the four above
 *   FGB_MB_LEAN     coupled, without pairs: the MMA lane keeps the instructions
 *                   between two stages' MMAs to a minimum (descriptors by one
 *                   add, next stage probed in the shadow of the last MMAs)
 *   FGB_MB_M64      the MMAs are 64 x 256 x 16 (MMA stream alone or independent)
 *   FGB_MB_STORE, FGB_MB_STORE_BULK128, FGB_MB_STORE_BULK512   in place of
 *                   the gather, the output stream of an epilogue: 32 KB per stage
 *                   from shared memory to random rows of `rows` (which these
 *                   modes overwrite), as 16-byte stores that cover four 128-byte
 *                   lines per warp instruction, as bulk async copies of 128 bytes,
 *                   or of whole 512-byte rows; not with GATHER, COUPLED or PAIR
 * stages_a / stages_b: ring depths of the two operands (1..6, together within
 * the shared memory of an SM).  issue_delay: cycles the MMA lane idles before
 * it issues a stage's MMAs (0 = none): how much instruction time between two
 * stages' MMAs the tensor pipe's queue hides.  One CTA per SM runs `iters` stages; *ms_out =
 * the launch's duration (CUDA events on `stream`; the call synchronises).
 * counters (host, [8], may be null) receive from CTA 0's MMA lane: cycles spent
 * waiting for the dense operand, number of such waits, the same two for the
 * gathered operand, total cycles of its loop.  The function allocates and frees
 * a few bytes of device memory. */
#define FGB_MB_TMA 1
#define FGB_MB_GATHER 2
#define FGB_MB_MMA 4
#define FGB_MB_COUPLED 8
#define FGB_MB_GATHER4 16
#define FGB_MB_PAIR 32
#define FGB_MB_LEAN 64
#define FGB_MB_M64 128
#define FGB_MB_STORE 256
#define FGB_MB_STORE_BULK128 512
#define FGB_MB_STORE_BULK512 1024
int fgb_microbench_pipeline(int mode, int stages_a, int stages_b, int iters, int issue_delay,
                            const void* rows, int64_t n_rows, int row_bytes,
                            const void* dense, int64_t dense_bytes,
                            float* ms_out, uint64_t* counters, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLEXGEMM_B200_H_ */
