/*
 * C ABI of libtritonblas_b200.so: the B200 (sm_100a) GEMM hot path behind the tritonBLAS Python API.
 *
 * Conventions
 *   - every entry point returns 0 on success or a positive TB_ERR_* code; tb_status_string() explains a code;
 *   - pointers are raw device pointers, sizes and strides are in ELEMENTS unless a name ends in _bytes;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised, unless stated;
 *   - the library neither allocates nor frees device memory: outputs and workspaces are caller-owned;
 *   - citations name the reference interface (path inside the tritonBLAS tree : line) an entry point stands in for.
 */
#ifndef TRITONBLAS_B200_H_
#define TRITONBLAS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum {
  TB_DTYPE_F16 = 0,
  TB_DTYPE_BF16 = 1,
  TB_DTYPE_F32 = 2,
  TB_DTYPE_E4M3 = 3,
  TB_DTYPE_E5M2 = 4,
  TB_DTYPE_U8 = 5, /* packed e2m1 pairs / e8m0 scale bytes */
  TB_DTYPE_F4 = 6, /* selector only: 4-bit e2m1 operand */
  TB_DTYPE_I8 = 7  /* signed 8-bit integers: int32 accumulate on the tensor cores, fp32 epilogue */
};

/* host-side error codes; codes >= 100 are device-side wait time-outs reported through tb_device_status() */
enum {
  TB_OK = 0,
  TB_ERR_INVALID = 1,     /* bad argument (shape, dtype, null pointer) */
  TB_ERR_UNSUPPORTED = 2, /* valid request this build has no kernel for */
  TB_ERR_ALIGNMENT = 3,   /* pointer or stride not usable by TMA and no fallback applies */
  TB_ERR_WORKSPACE = 4,   /* workspace missing or too small */
  TB_ERR_CUDA = 5,        /* a CUDA runtime / driver call failed; see tb_last_cuda_error() */
  TB_ERR_NO_DEVICE = 6
};

/* GEMM problem as the selector sees it. Replaces the argument list of
 * OrigamiMatmulSelector.__init__ (include/tritonblas/origami.py:98-112). */
typedef struct tb_problem {
  int32_t m, n, k;
  int32_t a_dtype, b_dtype, c_dtype;
  int32_t a_mn_major;    /* 1: A stored with M contiguous (reference "N" layout); 0: K contiguous */
  int32_t b_mn_major;    /* 1: B stored with N contiguous; 0: K contiguous */
  int32_t streamk;       /* 1: caller asked for stream-K scheduling */
  int32_t mx_block_size; /* 0, or 32 for MXFP4 */
  int32_t num_sms;       /* 0: all SMs of the device; else restrict the model and the grid to this many */
  int32_t device;
  int32_t max_halves;    /* 0: the model may pick wide tiles (tb_config.n_halves = 2); 1: narrow tiles only (what grouped
                            launches want) */
} tb_problem;

/* Launch configuration chosen by the analytical model. Replaces the attribute surface of the selector
 * (block_m/block_n/block_k/group_m/num_stages/sk_grid, include/tritonblas/origami.py:313-347) and the hybrid
 * split computed in streamk_matmul_lt (include/tritonblas/matmul.py:225-254). */
typedef struct tb_config {
  int32_t block_m;   /* output tile rows (128 per CTA, 256 for a CTA pair) */
  int32_t block_n;   /* output tile columns */
  int32_t block_k;   /* K elements per shared-memory stage */
  int32_t group_m;   /* tile-order swizzle: tiles_m grouped per column sweep */
  int32_t stages;    /* shared-memory ring depth */
  int32_t cta_pair;  /* 1: one CTA per tile; 2: two CTAs (one cluster) per tile */
  int32_t grid;      /* programs (CTAs or CTA pairs) of the data-parallel launch */
  int32_t sk_grid;   /* programs of the stream-K launch */
  int32_t num_sms;   /* SMs of the device */
  int32_t smem_bytes;
  int32_t tmem_cols;
  float predicted_us;     /* model estimate for the data-parallel schedule */
  float predicted_sk_us;  /* model estimate for the stream-K schedule */
  int32_t n_halves;  /* 1, or 2: a work tile is two block_n-wide accumulators side by side that share every A stage
                        (tile = block_m x 2*block_n; fewer L2 -> shared-memory bytes per flop, no cross-tile epilogue
                        overlap). 0 is read as 1. Ignored by stream-K launches; measured no gain for grouped launches. */
  int32_t swap_ab;   /* 1: the kernel computes C^T = B^T A^T (few rows of A: the weight matrix takes the 128-row side of
                        the tile); block_m/block_n then describe the swapped problem */
} tb_config;

/* One dense GEMM: C = cast( (A . B) [* a_scale[:,None]] [* b_scale[None,:]] [+ bias[None,:]] ).
 * Replaces persistent_matmul_lt / streamk_matmul_lt and the Triton kernels they launch
 * (include/tritonblas/matmul.py:69-366, kernels/persistent_gemm.py:26-126, kernels/streamk_gemm.py:7-384). */
enum { TB_EPILOGUE_NONE = 0, TB_EPILOGUE_SWIGLU = 1 };

typedef struct tb_gemm_args {
  int32_t m, n, k;
  int32_t a_dtype, b_dtype, c_dtype;
  const void* a; int64_t a_stride_m, a_stride_k;
  const void* b; int64_t b_stride_k, b_stride_n;
  void* c;       int64_t c_stride_m, c_stride_n;
  const float* a_scale;  /* (m,) fp32 contiguous or NULL */
  const float* b_scale;  /* (n,) fp32 contiguous or NULL */
  const void* bias;      /* (n,) or NULL */
  int64_t bias_stride; int32_t bias_dtype;
  int32_t allow_tf32;    /* fp32 operands: 1 = tensor-core tf32 products, 0 = exact fp32 products */
  int32_t streamk;       /* 0: data-parallel persistent; 1: hybrid stream-K */
  int32_t sk_grid;       /* >0 overrides the configuration's stream-K grid */
  void* workspace;       /* stream-K: partial tiles + flags; see tb_gemm_workspace_bytes() */
  int64_t workspace_bytes;
  uint32_t epoch;        /* stream-K: a value never used before on this workspace (start at 1, add 1 per launch;
                            the workspace must be zero-filled once when it is created) */
  /* Grouped (MoE) GEMM, tb_grouped_gemm only: group g multiplies rows [group_offsets[g], group_offsets[g+1]) of A
   * (m = total rows) by its own B_g, stored as rows [g*n, (g+1)*n) of a (num_groups*n, k) K-contiguous matrix, into the
   * same rows of C. group_offsets is a DEVICE array of num_groups + 1 ascending int32; the kernel clamps the offsets to
   * [0, m], so offsets that describe more than m rows lose their tail instead of reaching past A and C. */
  const int32_t* group_offsets;
  int32_t num_groups;
  /* Fused output fan-out (tb_gemm only): up to 7 further destinations with c's dtype, shape and strides — typically the
   * same buffer on peer GPUs, mapped into this process (CUDA IPC / symmetric memory). The epilogue stores every tile to c
   * and to each of them with ordinary stores, so the transfer over NVLink overlaps the remaining tiles' math; the caller
   * synchronises the ranks before the copies are read. HOST array of device pointers, or NULL. */
  void* const* c_copies;
  int32_t num_c_copies;
  /* Dynamic tile schedule, the reference's work_stealing=True (kernels/persistent_gemm_work_stealing.py:106-116,
   * config.py:104-121): DEVICE pointer to two uint32 words, zero when first used, or NULL for the static schedule. Every
   * program starts with its own first tile and takes the following ones from a shared counter, so programs that start
   * late (another kernel holds their SMs) take fewer tiles. The last program leaves both words zero again, so launches
   * that follow each other on one stream share the buffer without a reset; after a failed launch the caller zeroes it.
   * Ignored by stream-K launches (as the reference's a8w8 path does, matmul.py:387-388). */
  void* tile_counter;
  /* Fused activation of the epilogue. TB_EPILOGUE_NONE, or TB_EPILOGUE_SWIGLU: B has 2*n rows (per group), the first n the
   * gate projection and the next n the up projection, and C (n columns) receives silu(a.gate_j) * (a.up_j) computed in fp32
   * on the accumulators and cast once. For the MoE gate/up projection (no reference counterpart: the reference has no
   * grouped kernel; its dense contract of fp32 accumulation and one cast is kept). Needs K-contiguous operands, a 16-bit
   * row-major C with 16-byte aligned rows, n a multiple of 128, more than 128 rows, no scales or bias, the data-parallel
   * schedule; the library then runs CTA pairs whose accumulators hold 128 gate and 128 up columns side by side, so the
   * activation hides behind the next tile's main loop. TB_ERR_UNSUPPORTED otherwise. */
  int32_t epilogue_op;
  /* Bound of every device-side wait of this launch in milliseconds; 0 = the default of 2 s. A wait that runs out makes
   * the kernel record a TB_DEV_* code (tb_device_status) and return; nothing spins for ever (the reference's waits are
   * unbounded, kernels/streamk_gemm.py:295-300). */
  int32_t wait_timeout_ms;
  /* Measurement and test switches, 0 in production. Bit 1 (value 2): per-role cycle counters are written to the start of
   * `workspace` (148 x 16 int64: clocks spent waiting / issuing / draining per role in words 0-8, wall-clock stamps in ns of
   * kernel entry, dependency wait, first filled stage, last MMA, last store and exit in words 9, 10, 12-15). Bit 2 (value 4): stream-K programs never publish their partial tile, so the owners'
   * bounded waits run out (RESULTS ARE WRONG; the failure-path test uses it). Bit 3 (value 8): every work item walks K
   * forwards. */
  int32_t debug_flags;
  /* Row gather (tb_grouped_gemm only; no reference counterpart): DEVICE int32[m], or NULL. Row r of the grouped problem is
   * then row a_gather_index[r] of the matrix `a`, which has a_rows rows (a_stride_m apart, K contiguous, 16-bit elements,
   * base and row pitch 16-byte aligned); an entry outside [0, a_rows) reads as a row of zeros. The MoE gate/up projection
   * reads the tokens' rows in expert order straight from the activation matrix this way, with no gathered copy in between. */
  const int32_t* a_gather_index;
  int64_t a_rows;
  /* Fan-out of only the first tiles (tb_gemm with c_copies). 0: every tile goes to the copies. > 0: only tiles with index
   * below this do (the kernel enumerates tiles in waves, so these are the launch's first waves); the caller sends the rest
   * with tb_push_c_tiles, typically on another stream beside the next launch, whose first tiles have nothing to send yet. */
  int32_t c_copies_tile_limit;
  /* Operands that no work still in flight on the stream writes (weights): bit 0 = a, bit 1 = b. Launches are made with
   * programmatic stream serialization, so a CTA can be scheduled while the previous kernel of the stream is still
   * draining; it then starts filling its shared-memory ring with such an operand at once instead of waiting for that
   * kernel first (single-CTA tiles, static schedules; ignored elsewhere). Everything else, the other operand, scales,
   * bias and workspace included, is only touched after the wait. 0: no promise, nothing is read early. */
  int32_t static_operands;
} tb_gemm_args;

/* Fill `cfg` for `p`. Stands in for origami.select_config + OrigamiMatmulSelector._compute_sk_grid
 * (include/tritonblas/origami.py:232-247,349-416); the model itself is derived for B200, not transcribed. */
int tb_select(const tb_problem* p, tb_config* cfg);

/* Bytes of stream-K workspace a launch with `cfg` (and optional grid override) needs.
 * Stands in for the locks/P sizing of matmul_preamble (include/tritonblas/config.py:104-110). */
int64_t tb_gemm_workspace_bytes(const tb_config* cfg, int32_t sk_grid_override);

/* Enqueue one GEMM. `cfg` may be NULL (the library selects). */
int tb_gemm(const tb_gemm_args* args, const tb_config* cfg, void* stream);

/* Tiles of the data-parallel launch tb_gemm would make for (args, cfg): tb_gemm_tile_count gives their number (what
 * c_copies_tile_limit is measured against); tb_push_c_tiles copies tiles [first_tile, count) of args->c into every
 * args->c_copies[x], in the kernel's own tile order. For the tail of a launch made with c_copies_tile_limit = first_tile.
 * 16-byte aligned rows of a unit-stride C; not for stream-K, grouped or transposed (swap_ab) configurations. No reference
 * counterpart. */
int tb_gemm_tile_count(const tb_gemm_args* args, const tb_config* cfg);
int tb_push_c_tiles(const tb_gemm_args* args, const tb_config* cfg, int32_t first_tile, void* stream);

/* Stream-K GEMM for callers that cannot allocate device memory: a serving process that handed all of HBM to its own
 * arena at start-up, or a latency path on which cudaMalloc (which synchronises the whole device) is not allowed, has no
 * way to size and own the partial-tile workspace tb_gemm asks for. This entry point takes no workspace: flags and fp32
 * partial tiles live in an array that is part of the library image (4 KB + 10 MB per GPU that loads the library, held
 * until the process exits). It calls no allocator (no cudaMalloc / cudaFree, no torch); nothing else in the library does
 * either. It has no counterpart in the reference.
 *   - Same arguments and launch path as tb_gemm with streamk = 1; args->workspace / workspace_bytes / epoch /
 *     tile_counter are ignored. epilogue_op, group_offsets / num_groups and c_copies are not offered here
 *     (TB_ERR_UNSUPPORTED).
 *   - Limit: a launch that splits a tile keeps one fp32 partial tile per CTA, programs x 128 x block_n x 4 bytes (x2 for a
 *     CTA pair), which must fit 10 MB; a launch that needs more returns TB_ERR_WORKSPACE and tb_last_cuda_error() says by
 *     how much (lower args->sk_grid, or use tb_gemm). A launch whose grid divides its tile count splits nothing and is
 *     never refused.
 *   - The first call on a device looks up the device address of the built-in array; make that first call before any
 *     stream capture begins.
 *   - All calls on a device share the one array, which keeps the previous call's contents (the flags are cleared at the
 *     start of every call, on `stream`): two calls whose kernels overlap on the GPU (different streams) race.
 *   - prev_status, when not NULL, receives and clears the device's failure code (the word tb_device_status reads)
 *     recorded by earlier launches; reading it waits for `stream`. Pass NULL to stay asynchronous. */
int tb_gemm_streamk_builtin(const tb_gemm_args* args, const tb_config* cfg, void* stream, int32_t* prev_status);

/* Grouped GEMM over row groups of A (expert-parallel MoE projections). No reference counterpart: its semantics are the
 * dense contract of tb_gemm applied per group. A and every B_g must be K-contiguous; data-parallel schedule only. */
int tb_grouped_gemm(const tb_gemm_args* args, const tb_config* cfg, void* stream);

/* Memory-bound steps around the grouped MoE GEMMs (the reference has no MoE path, so no counterpart):
 *   tb_swiglu:      out[r, j] = silu(h[r, j]) * h[r, ffn + j] for h = [gate | up] (rows, 2*ffn); fp32 math, one cast.
 *   tb_moe_combine: out[t, :] = sum_k weights[t, k] * y[pos[t, k], :]; pos = row of y that holds the k-th expert output
 *                   of token t (int64, tokens x topk), weights fp32 (tokens x topk); fp32 accumulate in k order.
 * f16 / bf16 data, 16-byte aligned rows, ffn and hidden multiples of 8. */
int tb_swiglu(const void* h, int64_t h_row_stride, void* out, int64_t out_row_stride, int64_t rows, int32_t ffn,
              int32_t dtype, void* stream);
int tb_moe_combine(const void* y, int64_t y_row_stride, const int64_t* pos, const float* weights, void* out,
                   int64_t out_row_stride, int32_t tokens, int32_t topk, int32_t hidden, int32_t dtype, void* stream);
/*   tb_moe_gather_rows: out[i, :] = x[src_row[i], :] for i < n (token rows into expert-major order on one GPU); int64
 *                       indices, 16-byte aligned rows, hidden a multiple of 8 elements of 2 bytes. */
int tb_moe_gather_rows(const void* x, int64_t x_row_stride, const int64_t* src_row, void* out, int64_t out_row_stride,
                       int64_t n, int32_t hidden, void* stream);

/* Expert-parallel dispatch and combine over peer-mapped memory (each rank's receive / output buffer mapped into every
 * process, e.g. by CUDA IPC or torch symmetric memory), in place of all-to-all collectives. Ordinary loads and stores.
 *   tb_moe_dispatch_peers: for i < n, row src_token[i] of x is copied to row dest_row[i] of peer_bufs[dest_rank[i]];
 *                          rows outside [0, capacity_rows) are dropped and counted in *overflow_count (device int, may
 *                          be NULL).
 *   tb_moe_combine_peers:  out[t, :] = sum_k weights[t,k] * y_peers[pair_rank[t,k]][pair_row[t,k], :] (fp32, k order);
 *                          pairs whose row lies outside [0, capacity_rows), i.e. rows the dispatch dropped, add nothing.
 * peer_bufs / y_peers are HOST arrays of up to 8 device pointers; index arrays are device memory. The caller orders the
 * phases across ranks (barrier after dispatch, barrier before combine). No reference counterpart. */
int tb_moe_dispatch_peers(const void* x, int64_t x_row_stride, const int64_t* src_token, const int32_t* dest_rank,
                          const int64_t* dest_row, void* const* peer_bufs, int32_t num_peers, int64_t dest_row_stride,
                          int64_t capacity_rows, int32_t* overflow_count, int64_t n, int32_t hidden, int32_t dtype,
                          int32_t topk, void* stream);
int tb_moe_combine_peers(void* const* y_peers, int32_t num_peers, int64_t y_row_stride, const int32_t* pair_rank,
                         const int64_t* pair_row, const float* weights, void* out, int64_t out_row_stride, int32_t tokens,
                         int32_t topk, int32_t hidden, int32_t dtype, int64_t capacity_rows, void* stream);

/* Dispatch plan of the expert-parallel MoE step, computed on the device (no host synchronisation, no sort). No reference
 * counterpart. topk_ids: n_pairs expert ids of the flattened (token, k) pairs, int32 or int64 (ids_are_int64).
 * expert_place (device int32[num_experts], or NULL for the identity) gives every expert id its position q in the order
 * the experts are laid out over the ranks: position q lives on rank q / (num_experts / world) as that rank's local expert
 * q % (num_experts / world). A placement that spreads the popular experts evens out the rows per rank. Counts, offsets and
 * rows below are all in placement order.
 *   tb_moe_count: counts[q] = pairs routed to the expert at position q (counts, int32[num_experts], is cleared by the call).
 *   tb_moe_plan:  counts_all is int32[world][num_experts], every rank's counts (for one GPU: the counts themselves).
 *                 In its owner's receive buffer the experts follow each other in placement order
 *                 and inside an expert the source ranks follow each other. Writes, for every pair f of this rank,
 *                 pair_rank[f] (owner) and pair_row[f] (row in the owner's buffer; -1 for an id outside [0, num_experts)),
 *                 and group_offsets[num_experts / world + 1], the row offsets of this rank's own experts clamped to
 *                 capacity_rows. cursor is int32[num_experts] scratch (cleared by the call). The order of the rows inside
 *                 an expert is unspecified; num_experts <= 1024. row_token (world == 1 only, else NULL): int32[capacity_rows],
 *                 receives the source token (pair index / topk) of every row, the index tb_gemm_args.a_gather_index takes. */
int tb_moe_count(const void* topk_ids, int32_t ids_are_int64, int64_t n_pairs, int32_t num_experts,
                 const int32_t* expert_place, int32_t* counts, void* stream);
int tb_moe_plan(const void* topk_ids, int32_t ids_are_int64, int64_t n_pairs, int32_t num_experts, const int32_t* expert_place,
                int32_t world, int32_t rank, const int32_t* counts_all, int32_t* cursor, int64_t capacity_rows,
                int32_t* pair_rank, int64_t* pair_row, int32_t* group_offsets, int32_t* row_token, int32_t topk, void* stream);

/* Diagnostic: streams rows x row_bytes of a row-major matrix (pitch_bytes between rows) out of HBM with the access pattern
 * of the GEMM's K-major operand loader and drops the data: `programs` CTAs (one per SM), each keeping `stages` TMA boxes of
 * box_rows rows x 128 bytes in flight, row blocks dealt round-robin, K walked in 128-byte steps. Time it with events:
 * rows / box_rows * box_rows * row_bytes bytes per launch. row_bytes a multiple of 128, box_rows a multiple of 8 up to 256,
 * stages * box_rows * 128 bytes within 196 KB. Waits are bounded and report through tb_device_status. No reference
 * counterpart. */
int tb_tma_stream_probe(const void* base, int64_t rows, int64_t row_bytes, int64_t pitch_bytes, int32_t stages,
                        int32_t box_rows, int32_t programs, void* stream);

/* Diagnostic (no reference counterpart): stores `passes` times `rows` rows of `run_bytes` contiguous bytes each, `pitch_bytes`
 * apart, into dst (a local buffer, or a peer GPU's buffer mapped into this process) from `blocks` x `threads` threads with
 * 16-byte stores: the store pattern of an epilogue that pushes output tiles to other GPUs. Timing it gives the egress rate
 * that bounds the fused GEMM + all-gather and the MoE dispatch (python -m tritonblas_b200.peer_bandwidth). dst, pitch and
 * run 16-byte aligned; run_bytes below 512 must divide 512. dst needs rows * pitch_bytes bytes. */
int tb_peer_store_probe(void* dst, int64_t pitch_bytes, int32_t run_bytes, int64_t rows, int32_t blocks, int32_t threads,
                        int32_t passes, void* stream);

/* MXFP4 GEMM: C (m, n) = sum over 32-element K blocks of (A_e2m1 * 2^(sa-127)) . (B_e2m1 * 2^(sb-127)), fp32
 * accumulate, one cast. A is (m, k/2) bytes and B is (n, k/2) bytes, two e2m1 codes per byte (even element in the low
 * nibble), K contiguous, row strides in bytes (multiples of 16). Scales are e8m0 bytes in the "atom" arrangement the
 * tensor core's scale copy consumes (see tb_mxfp4_scales_to_atoms): set scales_in_atoms = 1. Runs on the block-scaled
 * tensor-core instruction. Replaces matmul_fp4 + the fp4_matmul kernel (include/tritonblas/matmul.py:519-625,
 * kernels/fp4_matmul.py:8-130). */
typedef struct tb_mxfp4_args {
  int32_t m, n, k;           /* k = number of 4-bit elements, a multiple of 32 */
  const void* a; int64_t a_row_stride;
  const void* b; int64_t b_row_stride;
  void* c; int64_t c_stride_m, c_stride_n; int32_t c_dtype;
  const void* a_scales;      /* tb_mxfp4_atoms_bytes(m, k) bytes */
  const void* b_scales;      /* tb_mxfp4_atoms_bytes(n, k) bytes */
  int32_t scales_in_atoms;   /* must be 1 */
  int32_t block_n;           /* 0 = library's choice; else 64, 128 or 192 */
  int32_t cta_pair;          /* 0 = library's choice; 1 or 2 */
  int32_t group_m;           /* 0 = library's choice */
} tb_mxfp4_args;
int tb_gemm_mxfp4(const tb_mxfp4_args* args, void* stream);

/* Scale bytes in "atom" order: [ceil(rows/128)][ceil(k/128)][512], the byte of (row r, K block j) inside its atom at
 * (r % 32) * 16 + ((r % 128) / 32) * 4 + (j % 4). Padding rows and blocks hold 127 (scale 1.0).
 * tb_mxfp4_atoms_bytes gives the buffer size; tb_mxfp4_scales_to_atoms re-arranges row-major (rows, k/32) scale bytes
 * (what the reference API passes, include/tritonblas/matmul.py:539-540) into it. */
int64_t tb_mxfp4_atoms_bytes(int64_t rows, int64_t k);
int tb_mxfp4_scales_to_atoms(const void* scales, int64_t scales_row_stride, int64_t rows, int64_t k, void* atoms,
                             void* stream);

/* MXFP4 block quantiser: x (rows, k) in f16/bf16/f32 with `x_row_stride` elements between rows, k % 32 == 0, to packed
 * e2m1 codes (rows, k/2) and e8m0 scale bytes (rows, k/32), both row-major with the given row strides in bytes.
 * hadamard = 0 replaces dynamic_mxfp4_quant / _dynamic_mxfp4_quant_kernel (include/tritonblas/utils.py:646-789) bit for
 * bit. hadamard = 1 first rotates every 32-element block by the Sylvester Hadamard matrix / sqrt(32) (fp32 butterflies,
 * strides 1,2,4,8,16, then one multiply); the reference has no such kernel. */
int tb_mxfp4_quant(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* codes,
                   int64_t codes_row_stride, void* scales, int64_t scales_row_stride, int32_t hadamard, void* stream);
/* Same, and additionally (when atoms != NULL) writes the scale bytes in atom order for tb_gemm_mxfp4; `scales` may then
 * be NULL. The atoms buffer must have been filled with 127 once (padding rows keep that value). */
int tb_mxfp4_quant_atoms(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* codes,
                         int64_t codes_row_stride, void* scales, int64_t scales_row_stride, void* atoms, int32_t hadamard,
                         void* stream);

/* Per-row symmetric FP8 e4m3 quantiser: scales[r] = max(amax(x[r,:]), 1e-8) / 448, q[r,:] = cast(x[r,:] * (1/scales[r])).
 * x is f16/bf16 (rows, k), k % 8 == 0. Rows of an activation are tokens, rows of a weight stored (N, K) are output
 * channels. Replaces the torch-op fixture quantize_tensor_per_channel(axis=1) (include/tritonblas/utils.py:340-377), same
 * arithmetic in the same order. */
int tb_fp8_quant_rows(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* q,
                      int64_t q_row_stride, float* scales, void* stream);

/* Reads (synchronously: waits for the device) and clears the per-device status word that kernels set when a bounded
 * wait gives up. 0 = no failure since the last call. No reference counterpart (its waits are unbounded,
 * kernels/streamk_gemm.py:295-300). */
int tb_device_status(int32_t device, int32_t* status_out);

/* Number of SMs, shared memory per block (opt-in) of a device. Stands in for origami.get_hardware_for_device
 * (include/tritonblas/origami.py:166). */
int tb_device_info(int32_t device, int32_t* num_sms, int32_t* smem_optin_bytes);

const char* tb_status_string(int code);
const char* tb_last_cuda_error(void);

/* Number of kernels this library has launched in this process (bench bookkeeping). */
int64_t tb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TRITONBLAS_B200_H_ */
