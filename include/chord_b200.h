/* chord_b200 - C ABI of the B200 (sm_100a) W4A16 MoE GEMM library.
 *
 * These are the entry points a binding of the reference library
 * (novitalabs/chord, package `chord_kernels`) calls in place of its own native
 * boundary: the torch custom ops `torch.ops.chord.launch_kernel`,
 * `launch_grouped_w4a16_masked`, `launch_grouped_w4a16_contiguous`
 * (chord_kernels/operator/csrc/launcher/launcher.cpp:52-158, 459-549, schemas
 * :605-630) and the repack kernel launch
 * (chord_kernels/operator/kernel/repack_weight.py:41-77).
 *
 * Conventions
 *  - Every pointer is a device pointer on the current CUDA device unless the
 *    parameter is documented as host memory.  The caller owns all buffers; the
 *    library never allocates, frees or synchronises (the single exception is
 *    chord_b200_repack_w4a16's optional range check, see there).
 *  - `stream` is a cudaStream_t passed as void*.
 *  - Functions return 0 on success, 1 for an argument/contract violation
 *    (bindings raise ValueError), 2 for an unsupported GPU and 3 for a CUDA
 *    failure (bindings raise RuntimeError).  chord_b200_last_error() returns
 *    the message of the calling thread's last failure.
 *  - Entry points may be called from several host threads.  The options set by
 *    chord_b200_set_option() are process-wide: a launch reads them under a lock and
 *    sees one consistent set, but which set a launch racing with a set_option call
 *    sees is unspecified.
 *  - Data formats (bit-exact with the reference):
 *      packed weight int32 [E, K/16, 2N], scale bf16 [E, K/32, N] as produced
 *      by pack_w4a16 (chord_kernels/operator/packing.py:55-138,
 *      include/humming/kernel/repack.cuh:8-121);
 *      N % 128 == 0, K % 64 == 0.
 */
#ifndef CHORD_B200_H_
#define CHORD_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Message of the calling thread's most recent failure ("" if none). */
const char* chord_b200_last_error(void);

/* Library build tag, e.g. "chord_b200 sm_100a". */
const char* chord_b200_version(void);

/* Process-wide tuning knobs, the counterpart of the reference's CHORD_W4A16_*
 * environment overrides (chord_kernels/operator/grouped/heuristics.py:32-39).
 * Unknown names and out-of-range values return 1.
 *   "x_load"          routed-row gather of `indexed` in the general kernel: 0 cp.async
 *                     helper warps (default), 1 TMA tile::gather4
 *   "dequant_groups"  2 (default) or 4 groups of four dequantising warps
 *   "issuers"         0 automatic (default); 1, 2 or 4 MMA-issuing threads
 *   "contiguous_tile" 0 automatic (default: 128-token tiles over two weight blocks
 *                     where "npair" applies, else 256); 128; 256 = merge neighbouring
 *                     128-row blocks of one expert into 256-token tiles
 *   "a_stages"        0 automatic (default); 2..7 depth of the tensor-memory operand ring
 *   "pregather"       1 (default) `indexed` with blocks of 64 rows or more first copies
 *                     the routed rows into slot order; 0 gathers inside the kernel
 *   "ksplit"          1 (default) single-issuer layouts give the second K half of tiles
 *                     of at most 128 tokens to a second issuer; 0 off
 *   "npair"           1 (default) tiles of at most 128 tokens with consecutive activation
 *                     rows span two neighbouring 128-row weight blocks, so that an
 *                     activation stage is fetched once per 256 weight rows; 0 one block
 *   "pair"            1 (default) tiles of more than 128 tokens with consecutive activation
 *                     rows and K >= 2048 run on clusters of two CTAs: one
 *                     tcgen05.mma.cta_group::2 stream multiplies two neighbouring 128-row
 *                     weight blocks (one per CTA) and each CTA loads half of the token rows
 *                     (no multicast); `contiguous` then takes two launches: each expert's
 *                     128-row blocks in pairs on 256-token tiles, the blocks left over
 *                     (single-block experts, the last block of an odd run) on 128-token
 *                     tiles; 0 off
 *   "decode_kernel"   1 (default) token tiles of at most 32 rows (indexed, masked) run
 *                     the warpgroup-per-worker kernel; 0 always the general kernel
 *   "max_stages"      0 as many shared-memory stages as fit (default), else a cap
 *   "grid_limit"      0 one CTA per SM (default), else at most this many CTAs
 *   "pdl"             1 launches of `indexed` and the SiLU*mul kernels carry the
 *                     programmatic stream-serialization attribute (programmatic
 *                     dependent launch, as the reference's enable_pdl does for its
 *                     grouped operators, launcher.cpp:440-451); 0 (default) off
 *   "lock_spins"      polls, 64 ns apart, a stream-K owner spends on its lock word
 *                     before it gives up and reports through `status` (default 2^22) */
int chord_b200_set_option(const char* name, int64_t value);

/* ---- packing: replaces repack_w4a16<kPacked> (repack.cuh:48-121) ----------
 * in : packed_input == 0: int32 codes [E, N, K], each in [0, 15];
 *      packed_input == 1: checkpoint words int32 [E, N, K/8], eight
 *      little-endian nibbles per word.
 * out: int32 [E, K/16, 2N].
 * range_flag: optional int32 device word; the kernel ORs 1 into it when a
 *      code lies outside [0, 15] (unpacked input only).  The reference checks
 *      this range on the host with torch.aminmax (packing.py:111-117). */
int chord_b200_repack_w4a16(const int32_t* in, int32_t* out, int64_t num_experts, int64_t n,
                            int64_t k, int packed_input, int32_t* range_flag, void* stream);

/* Replaces _pack_weight_scale (packing.py:45-52): bf16 [E, N, K/32] ->
 * bf16 [E, K/32, N] with out[e, g, 64c + j] = in[e, 64c + 8*(j%8) + j/8, g]. */
int chord_b200_permute_scale(const void* in, void* out, int64_t num_experts, int64_t n, int64_t k,
                             void* stream);

/* ---- schedule queries ------------------------------------------------------
 * Routing block size for `indexed` (replaces indexed_block_m /
 * select_indexed_config(...).block_m, chord_kernels/operator/api.py:300-315,
 * tuning.py:512-554).  Always a multiple of 8. */
int chord_b200_indexed_block_m(int64_t n, int64_t k, int64_t num_experts, int64_t routed_m);

/* Token-tile size the masked kernel uses for `expected_m` (replaces
 * _w4a16_masked_bm, chord_kernels/operator/grouped/heuristics.py:58-72). */
int chord_b200_masked_tile_m(int64_t expected_m);

/* Bytes of FP32 stream-K scratch a GEMM launch with this token tile needs on
 * the current device (the reference allocates it per launch inside its
 * launcher, launcher.cpp:110-123).  Returns < 0 on error. */
int64_t chord_b200_gemm_workspace_bytes(int64_t tile_tokens);

/* Bytes of scratch chord_b200_indexed wants for routing blocks of `block_m` rows,
 * `sorted_len` routing slots and reduction depth `k`: the stream-K scratch above plus,
 * for blocks of 64 rows or more, room for a copy of the routed activation rows in slot
 * order (sorted_len * k BF16), which lets the kernel load them as TMA boxes.  A caller
 * that passes only chord_b200_gemm_workspace_bytes() still gets a correct, slower
 * launch (rows gathered inside the kernel).  No counterpart in the reference, whose
 * launcher sizes its own scratch (launcher.cpp:110-123).  Returns < 0 on error. */
int64_t chord_b200_indexed_workspace_bytes(int64_t block_m, int64_t sorted_len, int64_t k);

/* Lock words a GEMM launch touches on the current device (all left zero).
 * The reference needs grid + grid/10 (launcher.cpp:95-109). */
int chord_b200_gemm_lock_words(void);

/* Host-side view of the tile schedule (no GPU needed): the segments CTA `cta` of a
 * `grid`-CTA launch works through for `tiles` output tiles of depth `k`.  Writes up
 * to `capacity` records of five int32 {tile, first k-block, end k-block, type
 * (0 whole tile, 1 stream-K owner, 2 stream-K contributor), peer (owner: number of
 * contributors; contributor: owner CTA)} and returns the number of segments, or
 * < 0 on a bad query.  Counterpart of the reference's Scheduler
 * (include/humming/scheduler.cuh:73-173), exposed so the split can be checked. */
int64_t chord_b200_schedule_segments(int64_t tiles, int64_t k, int64_t grid, int64_t cta,
                                     int32_t* out, int64_t capacity);

/* ---- indexed GEMM: replaces launch_kernel (launcher.cpp:52-158) -------------
 * out[id, :] = x[id / top_k, :] . dequant(W[expert_ids[block of id]])^T for every
 * id < m * top_k found in sorted_ids[0 .. *num_tokens_padded).
 *  x                 bf16 [m, k]
 *  sorted_ids        int32 [sorted_len]; blocks of block_m ids, valid prefix then sentinels
 *  expert_ids        int32 [expert_len]; expert of each block
 *  num_tokens_padded int32 [1], read on the device
 *  out               bf16 [m * top_k, n]; rows no id names are left untouched
 *  locks             int32 [num_locks] all zero on entry, all zero on exit
 *  workspace         scratch of chord_b200_indexed_workspace_bytes(block_m, sorted_len, k)
 *                    (at least chord_b200_gemm_workspace_bytes(block_m)), 16-byte aligned
 *  status            optional int32 word; a kernel that gives up on a bounded
 *                    wait ORs a nonzero code into it instead of hanging
 *  block_m           multiple of 8, at most 256 */
int chord_b200_indexed(const void* x, const int32_t* packed, const void* scale,
                       const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                       int64_t expert_len, const int32_t* num_tokens_padded, void* out,
                       int32_t* locks, int64_t num_locks, void* workspace, int64_t workspace_bytes,
                       int32_t* status, int64_t m, int64_t n, int64_t k, int64_t num_experts,
                       int64_t top_k, int64_t block_m, void* stream);

/* ---- gate_up GEMM with SiLU*mul in the epilogue -----------------------------------
 * No counterpart in the reference, which stops at the GEMM and leaves the activation to
 * its caller (docs/getting_started.md:5-14).  Same arguments as chord_b200_indexed for
 * a fused gate/up weight of N rows (gate rows first, then as many up rows: the w13
 * convention of tests/generators.py:419-420), but
 *   out[id, j] = bf16(silu(g) * u),  g = x[id / top_k] . W[e][j],  u = x[id / top_k] . W[e][N/2 + j]
 * with g and u taken from the FP32 accumulators, for j < N/2: out is bf16
 * [m * top_k, N/2] and the [m * top_k, N] intermediate never exists.  Each tile
 * computes a 128-row gate block and its up block side by side.
 * Available (chord_b200_gate_up_silu_supported() != 0) for routing blocks of at most 16
 * rows when K % 128 == 0, and for blocks of 64 to 128 rows; N % 256 == 0.  Otherwise
 * the call returns 1 and the caller runs chord_b200_indexed + chord_b200_silu_mul.
 * workspace: chord_b200_gate_up_silu_workspace_bytes(block_m, sorted_len, k). */
int chord_b200_indexed_gate_up_silu(const void* x, const int32_t* packed, const void* scale,
                                    const int32_t* sorted_ids, int64_t sorted_len,
                                    const int32_t* expert_ids, int64_t expert_len,
                                    const int32_t* num_tokens_padded, void* out, int32_t* locks,
                                    int64_t num_locks, void* workspace, int64_t workspace_bytes,
                                    int32_t* status, int64_t m, int64_t n, int64_t k,
                                    int64_t num_experts, int64_t top_k, int64_t block_m, void* stream);
int chord_b200_gate_up_silu_supported(int64_t n, int64_t k, int64_t block_m);
int64_t chord_b200_gate_up_silu_workspace_bytes(int64_t block_m, int64_t sorted_len, int64_t k);

/* ---- indexed GEMM with a table of output row addresses ----------------------------
 * No counterpart in the reference, whose epilogue stores row `id` at out + id * n
 * (include/humming/epilogue/gmem_writer.cuh:93-103).  Same operation and arguments as
 * chord_b200_indexed, except that the result of routed id goes to the BF16 row whose
 * address is out_rows[id] (a device array of m * top_k addresses, each 16-byte
 * aligned; a null entry drops the row).  The addresses may lie in another GPU's memory
 * that is mapped into this process: the expert-parallel layer uses this to let the
 * down projection store every result row straight into the result tensor of the GPU
 * the token came from (the combine step of the exchange, done by the epilogue's own
 * peer stores). */
int chord_b200_indexed_rows(const void* x, const int32_t* packed, const void* scale,
                            const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                            int64_t expert_len, const int32_t* num_tokens_padded, void* const* out_rows,
                            int32_t* locks, int64_t num_locks, void* workspace, int64_t workspace_bytes,
                            int32_t* status, int64_t m, int64_t n, int64_t k, int64_t num_experts,
                            int64_t top_k, int64_t block_m, void* stream);

/* ---- indexed GEMM over rows that are already in routing-slot order ----------------
 * No counterpart in the reference.  Same operation as chord_b200_indexed with top_k = 1,
 * for a caller that has placed the activation rows where the routing puts them: row s of
 * x (bf16 [m, k], m >= sorted_len) belongs to slot s, and sorted_ids[s] is s for a slot that
 * holds a row and any value >= m for padding.  The kernel then loads the rows of a block
 * as consecutive TMA boxes; nothing is gathered or copied.  The result of slot s goes to
 * out + s * n (out != null), or to the row whose address is out_rows[s] (out == null, as
 * chord_b200_indexed_rows); with fuse_silu != 0, w is a gate_up projection and out receives
 * silu(gate) * up, [m, n / 2] (as chord_b200_indexed_gate_up_silu, same support rules).
 * The expert-parallel layer receives its rows in this order (chord_b200_ep_dispatch). */
int chord_b200_indexed_slots(const void* x, const int32_t* packed, const void* scale,
                             const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                             int64_t expert_len, const int32_t* num_tokens_padded, void* out,
                             void* const* out_rows, int32_t* locks, int64_t num_locks, void* workspace,
                             int64_t workspace_bytes, int32_t* status, int64_t m, int64_t n, int64_t k,
                             int64_t num_experts, int64_t block_m, int fuse_silu, void* stream);

/* ---- indexed GEMM without a workspace argument ---------------------------------
 * No counterpart in the reference (its launcher always takes the stream-K scratch
 * from torch's allocator).  Same operation and arguments as chord_b200_indexed, but
 * the FP32 stream-K scratch is a fixed 5 MiB array inside the library image, so the
 * call allocates nothing on the device.  It is meant for hosts that must not call
 * cudaMalloc on the request path: a serving loop whose memory pool is sized and
 * frozen at start-up, a plugin running inside another process's CUDA context whose
 * allocator it may not touch, or code between the begin and end of a region in which
 * allocation is forbidden.
 *  - Limits: block_m <= 64 and at most 160 CTAs (one per SM); anything larger is
 *    refused with return code 1 and a message naming the limit.
 *  - Which kernel runs follows from what fits into the 5 MiB: with block_m <= 16 the
 *    decode kernel, as for chord_b200_indexed (results bit-equal to it).  With
 *    block_m 17..32 the decode kernel's one slot per warpgroup (9.7 MB on 148 SMs) does
 *    not fit, so the general kernel runs where chord_b200_indexed would run the decode
 *    kernel: same results within the output tolerance, not bit-equal, and slower.
 *    With block_m 33..64 there is no room for the slot-ordered copy of the routed
 *    rows, so they are gathered inside the kernel (slower than chord_b200_indexed
 *    with its full workspace).
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, once per device); make that first call outside any
 *    stream capture.
 *  - All calls on a device share the one array: calls that may overlap on the GPU
 *    (different streams without ordering) race on it, exactly as calls sharing
 *    `locks` do.  Nothing in it needs clearing between calls.
 *  - Every GPU that loads the library keeps the 5 MiB until the process exits. */
int chord_b200_indexed_static_scratch(const void* x, const int32_t* packed, const void* scale,
                                      const int32_t* sorted_ids, int64_t sorted_len,
                                      const int32_t* expert_ids, int64_t expert_len,
                                      const int32_t* num_tokens_padded, void* out, int32_t* locks,
                                      int64_t num_locks, int32_t* status, int64_t m, int64_t n,
                                      int64_t k, int64_t num_experts, int64_t top_k,
                                      int64_t block_m, void* stream);

/* ---- contiguous GEMM: replaces launch_grouped_w4a16_contiguous
 * (launcher.cpp:505-549) --------------------------------------------------------
 * out[r, :] = x[r, :] . dequant(W[m_indices[tile first row]])^T for every 128-row
 * tile whose first row has m_indices >= 0; other tiles are left untouched.  Inside
 * such a tile the rows after its last row with m_indices >= 0 (the padding the
 * contract requires to be zeroed) are written as zeros without being computed: what
 * the reference's kernel produces from their all-zero activations.
 *  x bf16 [m, k], m % 128 == 0; m_indices int32 [m]; out bf16 [m, n];
 *  enable_pdl != 0 launches with the programmatic stream-serialization attribute
 *  (launcher.cpp:440-451). */
int chord_b200_contiguous(const void* x, const int32_t* packed, const void* scale,
                          const int32_t* m_indices, void* out, int32_t* locks, int64_t num_locks,
                          void* workspace, int64_t workspace_bytes, int32_t* status, int64_t m,
                          int64_t n, int64_t k, int64_t num_experts, int enable_pdl, void* stream);

/* ---- masked GEMM: replaces launch_grouped_w4a16_masked (launcher.cpp:459-503) --
 * out[g, r, :] = x[g, r, :] . dequant(W[g])^T for r < masked_m[g]; other rows are
 * left untouched.
 *  x bf16 [num_groups, max_m, k]; masked_m int32 [num_groups];
 *  out bf16 [num_groups, max_m, n]; tile_m from chord_b200_masked_tile_m();
 *  enable_pdl as for chord_b200_contiguous. */
int chord_b200_masked(const void* x, const int32_t* packed, const void* scale,
                      const int32_t* masked_m, void* out, int32_t* locks, int64_t num_locks,
                      void* workspace, int64_t workspace_bytes, int32_t* status,
                      int64_t num_groups, int64_t max_m, int64_t n, int64_t k, int64_t tile_m,
                      int enable_pdl, void* stream);

/* ---- SiLU * mul between gate_up and down --------------------------------------
 * out[r, j] = silu(in[r, j]) * in[r, inter + j], in bf16 [rows, 2*inter], out bf16
 * [rows, inter].  The reference leaves this step to its caller; the gate-first
 * column order is the fused-w13 convention its shapes assume
 * (tests/generators.py:419-420). */
int chord_b200_silu_mul(const void* in, void* out, int64_t rows, int64_t inter, void* stream);

/* Same, but only for the rows named by the valid ids (< row_limit) among
 * sorted_ids[0 .. *num_tokens_padded): the rows `indexed` wrote. */
int chord_b200_silu_mul_routed(const void* in, void* out, const int32_t* sorted_ids,
                               int64_t sorted_len, const int32_t* num_tokens_padded,
                               int64_t row_limit, int64_t inter, void* stream);

/* ---- routing alignment (moe_align_block_size) -----------------------------------
 * CUDA form of the reference's align_routing_blocks (tests/generators.py:192-230):
 * topk_ids int32 [numel] holds global expert ids; routes to experts in
 * [expert_base, expert_base + num_experts) are sorted by expert (ids ascending
 * inside an expert) into blocks of block_m, padded with the sentinel `numel`.
 * Experts without routes emit no block.
 *  sorted_ids int32 [sorted_cap], expert_ids int32 [expert_cap] (local expert
 *  index), num_tokens_padded int32 [1].  Capacities must cover the worst case
 *  numel + num_experts * (block_m - 1) ids. */
int chord_b200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int64_t expert_base,
                                    int64_t num_experts, int64_t block_m, int32_t* sorted_ids,
                                    int64_t sorted_cap, int32_t* expert_ids, int64_t expert_cap,
                                    int32_t* num_tokens_padded, void* stream);

/* ---- expert-parallel exchange over peer memory -------------------------------------
 * No counterpart in the reference, which has no communication code ("EP routing may
 * carry only this rank's routes", docs/getting_started.md:21).  One process per GPU;
 * experts are split contiguously, rank r owning [r * experts_per_rank, (r + 1) *
 * experts_per_rank).  The host maps four buffers of every rank into every process
 * (symmetric memory, CUDA IPC) and passes device arrays of the `world` addresses as this
 * process sees them:
 *   peer_state     exchange state of chord_b200_ep_state_bytes() bytes, zeroed once
 *   peer_recv_x    bf16 [capacity, hidden]: routed activation rows arriving at the owner,
 *                  already in routing order: expert after expert, each expert's rows padded
 *                  to whole blocks of block_m slots (capacity = a multiple of block_m that
 *                  covers every route of every rank plus block_m - 1 slots per local expert)
 *   peer_recv_tag  int32 [capacity]: source rank << 24 | route of the row in each slot
 *   peer_routed    bf16 [routed_rows_per_rank, hidden]: result rows, route order
 * `epoch` is a counter every rank advances by one per layer call (1, 2, ...): flags
 * carry it, nothing is reset between calls.  The kernels use plain peer loads and
 * stores, no TMA and no multicast.  Every cross-GPU wait is bounded (about five
 * seconds); a wait that runs out ORs a bit into the `status` word at the end of the
 * state (256 counts, 512 rows, 1024 results, 2048 receive buffer too small) and the
 * kernel carries on with incomplete data instead of hanging.  At most 1024 experts over
 * all ranks.
 * One layer call, all on one stream:
 *   chord_b200_ep_plan      send_pos[i] = position of route i among this rank's routes to
 *                           the same expert (-1 for an expert outside all ranks);
 *                           publishes the per-expert counts to every peer
 *   chord_b200_ep_dispatch  waits for all counts, derives the first slot of this rank's rows
 *                           of every expert in its owner's buffers (inside an expert: source
 *                           rank after source rank), copies every route's row and tag
 *                           there, flags every peer
 *   chord_b200_ep_align     on the owner: waits for all rows; recv_count =
 *                           *num_tokens_padded = slots in use; sorted_ids[s] = s for a slot
 *                           that holds a row, capacity for padding; expert_ids per block;
 *                           row_ptr[s] = address in the source rank's peer_routed of the row
 *                           that receives slot s's result
 *   (gate_up + SiLU*mul = chord_b200_indexed_slots on recv_x with m = capacity and
 *    fuse_silu = 1; down = chord_b200_indexed_slots with out_rows = row_ptr: the rows are
 *    loaded where they landed, nothing is copied into slot order)
 *   chord_b200_ep_combine_signal   flags every peer: this owner's results are stored
 *   chord_b200_ep_combine_wait     returns (stream-ordered) once every owner has flagged */
int64_t chord_b200_ep_state_bytes(void);
int chord_b200_ep_plan(const int32_t* topk_ids, int64_t routes, int64_t experts_per_rank, int64_t world,
                       int64_t rank, int32_t* send_pos, void* const* peer_state, int64_t epoch,
                       void* stream);
int chord_b200_ep_dispatch(const void* x, const int32_t* topk_ids, const int32_t* send_pos, int64_t routes,
                           int64_t top_k, int64_t hidden, int64_t experts_per_rank, int64_t world,
                           int64_t rank, void* state, void* const* peer_state, void* const* peer_recv_x,
                           void* const* peer_recv_tag, int64_t capacity, int64_t block_m, int64_t epoch,
                           void* stream);
int chord_b200_ep_align(void* state, const int32_t* recv_tag, int64_t capacity, int64_t world, int64_t rank,
                        int64_t num_local_experts, int64_t block_m, int32_t* sorted_ids, int64_t sorted_cap,
                        int32_t* expert_ids, int64_t expert_cap, int32_t* num_tokens_padded,
                        int32_t* recv_count, void* const* peer_routed, int64_t routed_rows_per_rank,
                        int64_t hidden, void** row_ptr, int64_t epoch, void* stream);
int chord_b200_ep_combine_signal(void* const* peer_state, int64_t world, int64_t rank, int64_t epoch,
                                 void* stream);
int chord_b200_ep_combine_wait(void* state, int64_t world, int64_t epoch, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* CHORD_B200_H_ */
