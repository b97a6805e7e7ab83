/*
 * glsdm.h — C ABI of the B200-native transactional shared-memory operator.
 *
 * The reference project (kreasof-ai/GL-SDM) has no C ABI: its seam for this path is the
 * Python package projects/gl-sdm/src/gl_sdm/memory, which on its "urm" backend calls
 * exactly three native functions
 *   - gl_sdm/memory/backends/urm.py:109-122      routed_snapshot_read(values, scores, width)
 *   - gl_sdm/memory/backends/urm.py:49-82        snapshot_read(values, addresses, weights)
 *   - gl_sdm/memory/backends/commit.py:57-58     commit(memory, indices, deltas, keys)
 * Every entry point below cites the reference interface whose arithmetic it replaces.
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless a parameter says "host".
 *   - Nothing here allocates device memory unless stated; scratch is passed in as
 *     `workspace`, sized by the matching *_workspace_bytes() query.
 *   - Kernels are launched on `stream`; calls return after launch (asynchronous).
 *   - A call with rows == 0 returns GLSDM_OK without a launch; its array pointers may be null
 *     (an empty array has no storage).
 *   - The return value is a glsdm_status. Data-dependent failures (an address outside the
 *     bank) are reported through a caller-owned device word `device_status`, which the
 *     kernels OR error bits into; the caller zeroes it and reads it back when it wants.
 *   - A "row" of routing work is one (request, token, head) triple; rows are laid out
 *     [batch, token, head] row-major exactly as the reference's score tensor
 *     [B, T, H, 2*half] (gl_sdm/memory/routing.py:10-14).
 *   - A bank is [banks, heads, slots, dim] row-major (gl_sdm/memory/state.py:8-9), fp32 as
 *     in the reference or bf16 (extension). banks == 1 means one bank shared by the batch.
 */
#ifndef GLSDM_H_
#define GLSDM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* glsdm_stream_t; /* same type as cudaStream_t */

typedef enum {
  GLSDM_OK = 0,
  GLSDM_ERR_ARGUMENT = 1,    /* null pointer, negative size, misaligned pointer */
  GLSDM_ERR_UNSUPPORTED = 2, /* shape outside what the kernels cover (e.g. width > 32) */
  GLSDM_ERR_WORKSPACE = 3,   /* workspace smaller than *_workspace_bytes() */
  GLSDM_ERR_CUDA = 4,        /* a CUDA runtime call or launch failed */
  GLSDM_ERR_LIMIT = 5        /* size beyond a fixed built-in capacity */
} glsdm_status;

typedef enum { GLSDM_F32 = 0, GLSDM_BF16 = 1 } glsdm_dtype;

/* Bits OR-ed into *device_status by kernels. */
#define GLSDM_DEV_ADDRESS_OUT_OF_RANGE 1u
#define GLSDM_DEV_WAIT_EXPIRED 2u
#define GLSDM_DEV_LOG_NOT_ASCENDING 4u  /* an undo log whose addresses do not ascend (see glsdm_commit_undo) */

int glsdm_abi_version(void);
const char* glsdm_status_string(int status);
/* Message of the last CUDA error seen by this library on the calling thread (host string). */
const char* glsdm_last_cuda_error(void);
/* Number of kernels this library has launched in the process so far (host counter). */
uint64_t glsdm_kernel_launches(void);

/* Describes the bank a routed read gathers from. `values` points at slot `slot_lo` of
 * partition 0: a rank that owns slots [slot_lo, slot_hi) of every partition passes its
 * shard, whose partition stride is (slot_hi - slot_lo) rows. An unsharded bank has
 * slot_lo = 0, slot_hi = slots. Rows whose slot falls outside [slot_lo, slot_hi) add
 * nothing to the reading (partial read of a slot-sharded bank). */
typedef struct {
  const void* values;
  int dtype;        /* glsdm_dtype */
  int64_t banks;    /* requests holding their own bank, or 1 for a shared bank */
  int32_t heads;
  int64_t slots;    /* logical slots per (bank, head) partition; a perfect square for product keys */
  int32_t dim;      /* value width D */
  int64_t slot_lo;
  int64_t slot_hi;
} glsdm_bank;

/* Product-key routing, reference gl_sdm/memory/routing.py:10-26 (torch_routed_read, the
 * part before the row gather) and the route half of backends/urm.py:109-122.
 *   scores      [rows, 2*half] fp32; first half = left factor (high digit of the slot).
 *   width       routes requested; out_k = min(width, min(width, half)^2) are produced.
 *   out_index   [rows, out_k] int64 if index_i64 else int32, slot numbers ascending.
 *   out_weights [rows, out_k] fp32, softmax of the selected sums in that order.
 * Equal scores prefer the larger factor index / larger slot; -0.0 ties with +0.0. */
int glsdm_pk_select(const float* scores, int64_t rows, int32_t half, int32_t width,
                    void* out_index, int index_i64, float* out_weights, glsdm_stream_t stream);

/* Snapshot read with supplied routes, reference gl_sdm/memory/routing.py:27-28,31-42
 * (gather_rows + weighted sum), gl_sdm/memory/transactions.py:28-35 (read) and
 * backends/urm.py:49-82 (snapshot_read).
 *   index/weights [rows, width]; a row belongs to bank (row / rows_per_bank) when
 *   bank->banks > 1 and to head (row % heads).
 *   requests      optional [rows / heads] int64: the bank of each group of `heads` rows
 *                 (the token-clock API's request indirection, transactions.py:13-16);
 *                 NULL = derive the bank from rows_per_bank.
 *   out_read      [rows, dim] fp32. */
int glsdm_snapshot_read(const glsdm_bank* bank, const void* index, int index_i64,
                        const float* weights, const int64_t* requests, int64_t rows,
                        int64_t rows_per_bank, int32_t width, float* out_read,
                        uint32_t* device_status, glsdm_stream_t stream);

/* Fused route + read: reference gl_sdm/memory/routing.py:10-28 in one pass
 * (routed_snapshot_read, backends/urm.py:109-122). out_index / out_weights may be NULL when
 * the caller needs only the readings (the query read of global_layer.py:27). */
int glsdm_pk_select_read(const glsdm_bank* bank, const float* scores, int64_t rows,
                         int64_t rows_per_bank, int32_t half, int32_t width, float* out_read,
                         void* out_index, int index_i64, float* out_weights,
                         uint32_t* device_status, glsdm_stream_t stream);

/* Fused write proposal: write route + prediction read + row gather + delta + sort key.
 * Reference gl_sdm/layers/global_layer.py:41-54 with gl_sdm/runtime/dense.py:11-14
 * (proposal_delta) and gl_sdm/memory/routing.py:31-42.
 *   scores   [rows, 2*half] fp32 write-router factor scores
 *   target   [rows, dim] fp32 or bf16 (target_dtype)
 *   beta     [rows] fp32 (already sigmoid-ed), log_decay [rows] fp32 (<= 0)
 *   mass     [rows / heads] fp32 per token, or NULL for 1
 *   position of a row inside its commit chunk = chunk_offset + (row / heads) % tokens
 *   key      = address * (chunk_size * num_layers) + position * num_layers + layer_index
 *   out_addresses [rows*out_k] int64 flat bank rows ((bank*heads+head)*slots + slot)
 *   out_deltas    [rows*out_k, dim] fp32
 *   out_keys      [rows*out_k] int64 */
int glsdm_pk_propose(const glsdm_bank* bank, const float* scores, const void* target,
                     int target_dtype, const float* beta, const float* log_decay,
                     const float* mass, int64_t rows, int64_t rows_per_bank, int64_t tokens,
                     int32_t half, int32_t width, int64_t chunk_offset, int64_t chunk_size,
                     int32_t num_layers, int32_t layer_index, int64_t* out_addresses,
                     float* out_deltas, int64_t* out_keys, uint32_t* device_status,
                     glsdm_stream_t stream);

/* Backward of the routed read with compact bank gradients: reference autograd through
 * gl_sdm/memory/routing.py:19-28; native counterparts gl_sdm/memory/backends/token.py:69-82
 * (_route_backward) and :134-144 (_read_backward), which write a dense zero-filled bank
 * gradient per read. Here the bank gradient stays compact: one row per route.
 *   grad_out [rows, dim] fp32; grad_weights [rows, width] fp32 or NULL (gradient arriving at
 *   the returned softmax weights); index/weights [rows, width] as the forward returned them
 *   grad_scores [rows, 2*half] fp32, written whole (softmax backward scattered to the factors)
 *   grad_rows [rows*width, dim] fp32 = w_k * grad_out, out_addresses [rows*width] int64 flat
 *   bank rows: feed them to glsdm_commit on a zero (or accumulating) gradient bank. */
int glsdm_read_backward(const glsdm_bank* bank, const float* grad_out, const float* grad_weights,
                        const void* index, int index_i64,
                        const float* weights, int64_t rows, int64_t rows_per_bank, int32_t width,
                        int32_t half, float* grad_scores, float* grad_rows, int64_t* out_addresses,
                        glsdm_stream_t stream);

/* The same backward for a read of an OLDER bank version whose storage copy-free commits have
 * since updated in place (the reference plans gradients "back through updates" of compact
 * overlays, projects/gl-sdm/OPTIMIZATION_PLAN.md, "Represent commits as compact overlays";
 * the per-commit clone this replaces is gl_sdm/memory/transactions.py:96). Each route's row
 * is resolved as glsdm_overlay_read resolves it: from the first of the n_logs undo logs
 * (oldest commit first, host arrays of device pointers / sizes, n_logs <= GLSDM_MAX_UNDO_LOGS)
 * that holds its address, else from the bank. With n_logs = 0 it is glsdm_read_backward. */
int glsdm_read_backward_version(const glsdm_bank* bank, const float* grad_out, const float* grad_weights,
                                const void* index, int index_i64, const float* weights, int64_t rows,
                                int64_t rows_per_bank, int32_t width, int32_t half, int32_t n_logs,
                                const int64_t* const* log_addresses, const void* const* log_rows,
                                const int64_t* log_entries, float* grad_scores, float* grad_rows,
                                int64_t* out_addresses, glsdm_stream_t stream);

/* Backward of glsdm_pk_propose: reference autograd through gl_sdm/layers/global_layer.py:41-51
 * and gl_sdm/runtime/dense.py:11-14 (proposal_delta), i.e. through the write route's softmax
 * weights, the prediction read, the row gather and the delta expression, in one kernel.
 *   scores / target / beta / log_decay / mass   the forward's operands
 *   addresses    [rows*out_k] int64 as the forward returned them (the routes it chose)
 *   grad_deltas  [rows*out_k, dim] fp32, the gradient arriving at the delta rows
 *   log_*        undo logs of the copy-free commits applied to the bank since the forward
 *                (oldest first, as for glsdm_read_backward_version); n_logs = 0 if none
 *   grad_scores  [rows, 2*half] fp32 written whole; grad_target [rows, dim] fp32;
 *   grad_beta / grad_log_decay [rows] fp32 (beta as passed, i.e. after the sigmoid)
 *   grad_rows    [rows*out_k, dim] fp32 compact bank gradient, one row per route at
 *                addresses[i]: fold it into a bank with glsdm_commit
 * Rows of at most 256 values (GLSDM_ERR_UNSUPPORTED beyond); no gradient for mass. */
int glsdm_pk_propose_backward(const glsdm_bank* bank, const float* scores, const void* target,
                              int target_dtype, const float* beta, const float* log_decay,
                              const float* mass, const int64_t* addresses, const float* grad_deltas,
                              int64_t rows, int64_t rows_per_bank, int32_t half, int32_t width,
                              int32_t n_logs, const int64_t* const* log_addresses,
                              const void* const* log_rows, const int64_t* log_entries,
                              float* grad_scores, float* grad_target, float* grad_beta,
                              float* grad_log_decay, float* grad_rows, glsdm_stream_t stream);

/* Row gather out[n, :] = flat[addresses[n], :] in the bank's dtype, reference
 * gl_sdm/memory/routing.py:37-42 (gather_rows), gl_sdm/memory/transactions.py:19-25
 * (selected) and gl_sdm/memory/backends/primitives.py:14-20 (_gather). */
int glsdm_gather_rows(const void* flat, int dtype, int64_t bank_rows, int32_t dim,
                      const int64_t* addresses, int64_t count, void* out,
                      uint32_t* device_status, glsdm_stream_t stream);

/* Token-clock write proposal, reference gl_sdm/memory/transactions.py:38-59 and
 * gl_sdm/memory/backends/token.py:180-203 (_propose_forward).
 *   requests [rows/heads] int64, index/weights [rows, width], target [rows, dim] fp32,
 *   beta/log_decay [rows] fp32, mass [rows/heads] fp32
 *   out_addresses [rows*width] int64 flat bank rows, out_deltas [rows*width, dim] fp32 */
int glsdm_token_propose(const glsdm_bank* bank, const int64_t* requests, const void* index,
                        int index_i64, const float* weights, const float* target,
                        const float* beta, const float* log_decay, const float* mass,
                        int64_t rows, int32_t width, int64_t* out_addresses, float* out_deltas,
                        uint32_t* device_status, glsdm_stream_t stream);

/* Slot-sharded write proposal (no counterpart in the reference, which is single-GPU; the
 * arithmetic is gl_sdm/runtime/dense.py:11-14 split between token owner and slot owner).
 * glsdm_write_error, on the token's rank:
 *   out_error [rows, dim] = beta * (target - exp(log_decay) * prediction), out_decay_m1 [rows]
 * glsdm_shard_offsets, on every rank for the all-gathered routes index [rows, width] int32:
 *   offsets [rows + 1] = exclusive prefix of the number of routes per row whose slot is in
 *   [slot_lo, slot_hi); offsets[rows] = this rank's entry count
 * glsdm_shard_propose, on the slot's rank: for each owned route, in (row, route) order,
 *   delta = mass * (decay_m1 * row + w * error), address = head * slots + slot and the key
 *   of glsdm_pk_propose; `bank` is this rank's shard of one shared bank (banks == 1);
 *   out_addresses are rows of that shard, out_keys use the bank-wide address.
 * glsdm_shard_read: partial reading of this rank's shard for all-gathered int32 routes.
 * Blocked addressing (all three): row r lives in block r / block_rows; consecutive blocks are
 * `*_stride` elements apart (the per-rank pieces of an all-gather). Within an error block the
 * [block_rows, dim] error rows are followed by the block's decay_m1 values; `decay_m1` points at
 * the first block's decay values, `error` at its first row. */
int glsdm_shard_read(const glsdm_bank* bank, const int32_t* index, const float* weights,
                     int64_t rows, int64_t block_rows, int64_t block_stride, int32_t width,
                     float* out_partial, uint32_t* device_status, glsdm_stream_t stream);
int glsdm_write_error(const float* prediction, const void* target, int target_dtype,
                      const float* beta, const float* log_decay, int64_t rows, int32_t dim,
                      float* out_error, float* out_decay_m1, glsdm_stream_t stream);
int glsdm_shard_offsets(const int32_t* index, int64_t rows, int64_t block_rows,
                        int64_t block_stride, int32_t width, int64_t slot_lo, int64_t slot_hi,
                        uint32_t* offsets, glsdm_stream_t stream);
int glsdm_shard_propose(const glsdm_bank* bank, const int32_t* index, const float* weights,
                        const float* error, const float* decay_m1, const float* mass,
                        const uint32_t* offsets, int64_t rows, int64_t block_rows,
                        int64_t route_stride, int64_t error_stride, int64_t tokens, int32_t width,
                        int64_t chunk_offset, int64_t chunk_size, int32_t num_layers,
                        int32_t layer_index, int64_t* out_addresses, float* out_deltas,
                        int64_t* out_keys, glsdm_stream_t stream);

/* Buffered commit: stable sort of the entries by key, per-address fp32 sum in that order,
 * one read-modify-write per touched bank row, no float atomics. Reference
 * gl_sdm/memory/transactions.py:69-97 (torch path) and backends/commit.py:12-58 (Triton).
 *   values_in   bank rows [bank_rows, dim] (dtype), first row = flat address row_base
 *   values_out  NULL or == values_in: update in place; otherwise the whole bank is copied
 *               to values_out first and values_in is left untouched (functional commit)
 *   addresses   [entries] int64 flat bank rows; rows outside [row_base, row_base+bank_rows)
 *               set GLSDM_DEV_ADDRESS_OUT_OF_RANGE and are dropped
 *   deltas      [entries, dim] fp32
 *   keys        [entries] int64 or NULL (= sort by address, arrival order within it)
 *   key_bits    number of low key bits that can be non-zero, 0 = all 64
 * Segments no longer than 256 entries are summed strictly left to right; longer ones in
 * 256-entry blocks whose partial sums are then added left to right. */
size_t glsdm_commit_workspace_bytes(int64_t entries, int32_t dim);
int glsdm_commit(const void* values_in, void* values_out, int dtype, int64_t row_base,
                 int64_t bank_rows, int32_t dim, const int64_t* addresses, const float* deltas,
                 const int64_t* keys, int64_t entries, int32_t key_bits, void* workspace,
                 size_t workspace_bytes, uint32_t* device_status, glsdm_stream_t stream);

/* Copy-free versioned commit ("overlay" commit). The reference keeps an old snapshot valid by
 * cloning the whole bank at every commit (gl_sdm/memory/transactions.py:96 index_copy,
 * gl_sdm/memory/state.py:61-62) and plans touched-row overlays instead
 * (OPTIMIZATION_PLAN.md, "Represent commits as compact overlays"). Here the bank is updated
 * in place and the commit writes an UNDO LOG: for every touched address, the row it held
 * before. An older version is then the current bank with the logs of all later commits
 * played back, oldest log winning.
 *   glsdm_commit_undo   as glsdm_commit in place, plus
 *     undo_addresses [entries] int64   the entries' addresses in KEY order (runs of equal
 *                                      addresses); valid after the call. glsdm_overlay_read
 *                                      searches this array by bisection, so the keys of an
 *                                      overlay commit must be monotone in the address (the
 *                                      reference's keys address*(C*L) + position*L + layer
 *                                      are; so is sorting by the address itself). A log whose
 *                                      addresses descend anywhere sets
 *                                      GLSDM_DEV_LOG_NOT_ASCENDING; glsdm_undo_apply does not
 *                                      depend on the order and stays correct
 *     undo_rows      [entries, dim]    bank dtype; position p holds the old row of
 *                                      undo_addresses[p] iff p is the first of its run
 *   glsdm_undo_apply    writes every logged old row back into the bank (materialises the
 *                       previous version in `values`, e.g. in a copy of the bank)
 *   glsdm_overlay_read  snapshot_read of an OLD version: each route's row is taken from the
 *                       first of the n_logs logs (given oldest commit first) that holds its
 *                       address, else from the bank. log_* are HOST arrays of n_logs device
 *                       pointers / sizes; n_logs <= GLSDM_MAX_UNDO_LOGS. Unsharded banks only.
 *                       With no logs it returns exactly what glsdm_snapshot_read returns. */
#define GLSDM_MAX_UNDO_LOGS 8
int glsdm_commit_undo(void* values, int dtype, int64_t row_base, int64_t bank_rows, int32_t dim,
                      const int64_t* addresses, const float* deltas, const int64_t* keys,
                      int64_t entries, int32_t key_bits, void* workspace, size_t workspace_bytes,
                      int64_t* undo_addresses, void* undo_rows, uint32_t* device_status,
                      glsdm_stream_t stream);
int glsdm_undo_apply(void* values, int dtype, int64_t row_base, int64_t bank_rows, int32_t dim,
                     const int64_t* undo_addresses, const void* undo_rows, int64_t entries,
                     glsdm_stream_t stream);
int glsdm_overlay_read(const glsdm_bank* bank, const void* index, int index_i64,
                       const float* weights, int64_t rows, int64_t rows_per_bank, int32_t width,
                       int32_t n_logs, const int64_t* const* log_addresses,
                       const void* const* log_rows, const int64_t* log_entries, float* out_read,
                       uint32_t* device_status, glsdm_stream_t stream);

/* Commit of a proposal in factored form: the delta rows
 *   delta_k = mass * ((decay - 1) * row_k + w_k * err),  err = beta * (target - decay * prediction)
 * (gl_sdm/runtime/dense.py:11-14; entries and keys of gl_sdm/layers/global_layer.py:44-54) are
 * never written out. The caller passes what they are made of — the write routes, the per-token
 * error rows and decay-1 of glsdm_write_error — and the reducer rebuilds each delta in registers
 * from the bank row it is updating. Same sums in the same order as glsdm_shard_propose /
 * glsdm_pk_propose followed by glsdm_commit in place: the banks come out bit-identical.
 *   bank          the shard to update in place ([1, heads, local slots, dim], slot range set)
 *   index/weights write routes as for glsdm_shard_propose (blocks of block_rows rows,
 *                 route_stride elements apart; one block: block_rows = rows)
 *   error         per block: [block_rows, dim] error rows then [block_rows] decay-1 values,
 *                 error_stride floats per block
 *   offsets       glsdm_shard_offsets of the same routes, entries = its total; or NULL for an
 *                 unsharded bank: every route is an entry, entries = rows * width (no host
 *                 synchronisation needed); rows must then be whole sequences of `tokens`
 *                 tokens x heads (rows laid out [sequence, token, head])
 *   workspace     glsdm_commit_factored_workspace_bytes(entries, dim), 256-byte aligned */
size_t glsdm_commit_factored_workspace_bytes(int64_t entries, int32_t dim);
int glsdm_commit_factored(const glsdm_bank* bank, const int32_t* index, const float* weights,
                          const float* error, const float* mass, const uint32_t* offsets,
                          int64_t entries, int64_t rows, int64_t block_rows, int64_t route_stride,
                          int64_t error_stride, int64_t tokens, int32_t width, int64_t chunk_offset,
                          int64_t chunk_size, int32_t num_layers, int32_t layer_index,
                          int32_t key_bits, void* workspace, size_t workspace_bytes,
                          uint32_t* device_status, glsdm_stream_t stream);
/* The same in two steps, so that the first can overlap other work that still reads the bank:
 *   GLSDM_COMMIT_ORDER  entries, sort and gather into the workspace (reads routes and errors,
 *                       touches neither the bank nor anything the caller owns)
 *   GLSDM_COMMIT_APPLY  segmented sums and the row updates, from the workspace as ORDER left it
 * Pass both bits for the one-call behaviour. Between the two calls the workspace, routes and
 * error array must stay as they were; the caller orders the streams (ORDER before APPLY). */
#define GLSDM_COMMIT_ORDER 1
#define GLSDM_COMMIT_APPLY 2
int glsdm_commit_factored_phased(const glsdm_bank* bank, const int32_t* index, const float* weights,
                                 const float* error, const float* mass, const uint32_t* offsets,
                                 int64_t entries, int64_t rows, int64_t block_rows, int64_t route_stride,
                                 int64_t error_stride, int64_t tokens, int32_t width, int64_t chunk_offset,
                                 int64_t chunk_size, int32_t num_layers, int32_t layer_index,
                                 int32_t key_bits, int32_t phases, void* workspace, size_t workspace_bytes,
                                 uint32_t* device_status, glsdm_stream_t stream);

/* How glsdm_commit_factored treats rows that a single entry writes (dense numbering only):
 * 1 = such rows are found with two bit maps over the addresses and updated straight from the
 * routes, only the entries of shared addresses are sorted; 0 = every entry is sorted;
 * -1 (default) = 1 when the commit is large and sparse enough for it to pay (at least
 * 786,432 entries, four bank rows per entry), else 0. Any other value only queries. Returns the
 * previous setting. The committed bank is bit-identical whichever runs. */
int glsdm_commit_factored_mode(int mode);

/* Commit for hosts that cannot provide a workspace. It has no counterpart in the reference
 * (whose commit allocates freely through PyTorch). Same arguments and result as glsdm_commit,
 * minus the workspace: the sort/reduce scratch is a 4 MiB array built into the library's
 * device image, held by every GPU that loads the library until the process exits. Meant for
 * plain C/C++ embedders without a tensor allocator, and for serving loops that must keep
 * cudaMalloc/cudaFree (which synchronise the whole device) off their request path. This call
 * allocates nothing and frees nothing.
 *   Limits: entries <= glsdm_commit_static_max_entries() (65536) and dim <= 256; larger
 *   requests return GLSDM_ERR_LIMIT and touch nothing.
 *   The first call on each device looks up the array's address (cudaGetSymbolAddress) with
 *   that device current; make that first call before any stream capture begins.
 *   All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *   (different streams without an ordering between them) race and corrupt each other's
 *   commit. Issue them on one stream, or order the streams with events. The calls must also
 *   be serialised on the HOST: a commit is a dozen launches and a memset, and two host threads
 *   that enqueue on the same stream interleave theirs. One enqueuing thread at a time. */
int glsdm_commit_static(const void* values_in, void* values_out, int dtype, int64_t row_base,
                        int64_t bank_rows, int32_t dim, const int64_t* addresses,
                        const float* deltas, const int64_t* keys, int64_t entries, int32_t key_bits,
                        uint32_t* device_status, glsdm_stream_t stream);
int64_t glsdm_commit_static_max_entries(void);

/* The bounded wait of the commit's chained kernels, on its own (a diagnostic with no
 * counterpart in the reference). One thread sums the 64-bit chain words [0, position) exactly
 * as a sort tile or a compaction block does: a word whose top two bits are 0 has not been
 * published yet and is polled, at most 2^20 times (about a second); then the kernel gives up,
 * sets GLSDM_DEV_WAIT_EXPIRED in *device_status and RETURNS - it never spins for ever and
 * never traps, so the context stays usable. Words are (kind << 62 | 1 << 56 | count) with
 * kind 1 = count of one block, 2 = count of that block and all before it. *out_count
 * receives the sum that was reached. Passing zeroed words shows how a kernel whose
 * predecessor never arrives ends. */
int glsdm_wait_probe(const void* words, int64_t position, uint32_t* device_status, uint32_t* out_count,
                     glsdm_stream_t stream);

/* Dense-key routing (flat keys): scores = queries x keys^T on the tensor cores, fused with
 * a running per-row top-k, so the [rows, slots] score matrix is never stored. The
 * reference has no per-slot key tensor; its nearest interface is the score GEMM of
 * gl_sdm/layers/global_layer.py:26 followed by routing.py:21-26 (tie rule, softmax).
 *   queries [rows, dk] bf16, keys [slots, dk] bf16 (this rank's shard), dk in {64,128}
 *   col_base  global slot number of keys row 0
 *   out_score [rows, width] fp32 and out_slot [rows, width] int32: the `width` best
 *   (score, slot) pairs of this shard, best first; ties prefer the larger slot.
 *   NaN scores (only possible when a query or key already holds NaN or infinities) are never
 *   candidates: a row keeps its `width` largest scores that are not NaN, +inf first, and a
 *   row with fewer than `width` of them pads its list with (score -inf, slot -1), which
 *   glsdm_topk_merge ranks below every real candidate. (The product-key entry points follow
 *   the reference's sort order instead, NaN above +inf: their scores are caller data.) */
size_t glsdm_score_topk_workspace_bytes(int64_t rows, int64_t slots, int32_t dk, int32_t width);
int glsdm_score_topk(const void* queries, const void* keys, int64_t rows, int64_t slots,
                     int32_t dk, int32_t width, int64_t col_base, float* out_score,
                     int32_t* out_slot, void* workspace, size_t workspace_bytes,
                     uint32_t* device_status, glsdm_stream_t stream);

/* Choose the kernel behind glsdm_score_topk: 2 = one CTA per 128 rows, key tiles of 256 slots,
 * 128x256x16 MMAs (default); 0 = one CTA per 256 rows, key tiles of 128 slots, 128x128x16 MMAs.
 * Any other value only queries. Returns the previous setting. Same results whichever runs. */
int glsdm_score_topk_variant(int which);
/* The work decomposition glsdm_score_topk would use (host arithmetic only, no GPU needed):
 * out[8] = row blocks with uniform parts, parts, key tiles per part, key tiles in all, row
 * blocks of the last wave that are cut further, their parts, key tiles per such part, rows per
 * block. Every (row block, key tile) pair belongs to exactly one unit. */
int glsdm_score_topk_plan(int64_t rows, int64_t slots, int32_t width, int32_t which, int32_t sms,
                          int32_t* out);

/* The same with row pitches (in elements, multiples of 8): a query matrix whose rows hold
 * several sub-queries, e.g. the two halves of a product-key query. */
int glsdm_score_topk_pitched(const void* queries, int64_t query_pitch, const void* keys,
                             int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                             int64_t col_base, float* out_score, int32_t* out_slot, void* workspace,
                             size_t workspace_bytes, uint32_t* device_status, glsdm_stream_t stream);

/* The same routing with a lower bound per row: row_floor [rows] fp32 (or NULL) holds, for every
 * query row, a score that the row's width-th best score OVER ALL SLOTS OF THE BANK is known to
 * reach - e.g. the width-th best another shard has already found. Candidates below it are
 * never kept, so a shard whose slots cannot compete does little list work; a row's list may
 * then come back shorter than width (padded with (-inf, slot -1)), which the candidate merge
 * accepts. Scores equal to the bound are kept, so ties are decided as without it. With the
 * true bound the merged routes are identical to those of the unbounded call. */
int glsdm_score_topk_bounded(const void* queries, int64_t query_pitch, const void* keys,
                             int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                             int64_t col_base, const float* row_floor, float* out_score,
                             int32_t* out_slot, void* workspace, size_t workspace_bytes,
                             uint32_t* device_status, glsdm_stream_t stream);

/* The same with the bounds exchanged between the shards of a slot-sharded bank WHILE their
 * kernels run (no counterpart in the reference, which is single-GPU). Every shard scores the
 * same query rows; a streaming top-k spends about width * (1 + ln(slots / width)) list
 * insertions per row before its threshold is tight, whatever the shard size, so R shards pay
 * that R times - unless a shard that reaches a row later starts from what the others found.
 *   floor_in    [floor_sources][rows] fp32 in THIS GPU's memory, -inf where nothing is known:
 *               peers store into it while this call runs; a unit reads its rows when it starts
 *   floor_out   HOST array of floor_peers device pointers (<= 7), each [rows] fp32: this
 *               shard's row in a peer's floor_in (peer memory, plain stores); when a unit ends,
 *               the width-th best score of each of its rows is stored there
 *   row_shift   rows are named (row + row_shift) % rows in floor_in / floor_out: give each
 *               shard a rotated copy of the queries so that they walk the rows in different
 *               orders and most rows are first finished by somebody else
 * Nobody waits for anybody: a bound that has not arrived is a missed saving, nothing more, and
 * a stale bound of the SAME call is still a bound. The caller must make sure that nothing of
 * an earlier call (other queries) is left in floor_in when this call starts, on every shard. */
int glsdm_score_topk_shared(const void* queries, int64_t query_pitch, const void* keys,
                            int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                            int64_t col_base, const float* row_floor, int64_t row_shift,
                            const float* floor_in, int32_t floor_sources, float* const* floor_out,
                            int32_t floor_peers, float* out_score, int32_t* out_slot, void* workspace,
                            size_t workspace_bytes, uint32_t* device_status, glsdm_stream_t stream);

/* Product-key routing from per-factor candidate lists: second stage of
 * gl_sdm/memory/routing.py:19-26 (candidate sums, selection, canonical order, softmax). The
 * lists [rows, min(width, half)] (score, factor index; best first) are what two
 * glsdm_score_topk calls produce for queries x sub-key codebooks [half, dk/2], so the factor
 * score matrix [rows, 2*half] that gl_sdm/layers/global_layer.py:26 materialises is never
 * written. out_index / out_weights as in glsdm_pk_select. */
int glsdm_pk_combine(const float* left_score, const int32_t* left_index, const float* right_score,
                     const int32_t* right_index, int64_t rows, int32_t half, int32_t width,
                     void* out_index, int index_i64, float* out_weights, glsdm_stream_t stream);

/* Merge per-shard candidates into the global routes (tie rule and softmax of
 * gl_sdm/memory/routing.py:21-26 applied to `parts` candidate lists per row).
 *   cand_score / cand_slot [parts, rows, width]; out_index ascending, out_weights softmax. */
int glsdm_topk_merge(const float* cand_score, const int32_t* cand_slot, int32_t parts,
                     int64_t rows, int32_t width, void* out_index, int index_i64,
                     float* out_weights, glsdm_stream_t stream);
/* The same with the parts' lists part_stride elements apart in both arrays (>= rows*width),
 * e.g. the receive buffer of one all-gather that carries a rank's scores and slots together. */
int glsdm_topk_merge_strided(const float* cand_score, const int32_t* cand_slot, int32_t parts,
                             int64_t part_stride, int64_t rows, int32_t width, void* out_index,
                             int index_i64, float* out_weights, glsdm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GLSDM_H_ */
