/*
 * b200q — GGUF block-quantized (Q8_0 / Q4_K / Q6_K) weight x activation product for
 * NVIDIA B200 (sm_100a).  C ABI: plain pointers and sizes, no exceptions cross it.
 *
 * What this boundary replaces in the reference engine.  The reference (Rust) never sees
 * a matmul: every attention QKV/O and MLP gate/up/down projection runs inside
 *     context.decode(batch)            inference/crates/icn-engine/src/lib.rs:2264
 * of its llama.cpp bindings, with weights placed on the device by
 *     LlamaModel::load_from_file       inference/crates/icn-engine/src/lib.rs:972
 * and multi-GPU placement declared by SplitMode / tensor_split
 *     inference/crates/icn-contracts/src/lib.rs:122-124,200-205
 *     inference/crates/icn-hardware/src/lib.rs:2568-2590.
 * The entry points below are what an FFI crate for that path would bind: a context per
 * device (one executor thread owns it, as design/inference/engine.md:49-50 requires of native
 * state), weight handles that stay resident like a loaded model, and one projection call
 * whose activation row count M is `batch.n_tokens()` (1 for decode, 1 + n_draft for
 * speculative verify, up to n_ubatch = 512 and beyond for prefill).
 *
 * Conventions
 *   - every function returns b200q_status (0 = OK); out-parameters come last;
 *   - handles are opaque; the library owns device memory until *_destroy;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - a b200q_ctx is used by one thread at a time; distinct contexts may be used from distinct
 *     threads (the library's one-time set-up is thread-safe);
 *   - calls are stream-ordered: each enqueues on the stream it is given and returns.  The scratch a
 *     context owns (fp16 activation copy, partial sums, dependency counters) is shared by all its
 *     b200q_matmul* calls, so keep one context's calls on one stream or order them with events;
 *     a plan owns its scratch, but two runs of one plan must not overlap.  The first call with a
 *     larger M x K may allocate: make it before any stream capture;
 *   - weights are W[N][K] in GGUF order: N output rows, each K/blk consecutive packed blocks;
 *   - activations X[M][K] and outputs Y[M][N] are row-major with leading dimensions in elements.
 *   - there is no CPU fallback: without a CUDA device every compute call fails with
 *     B200Q_ERR_BACKEND.
 */
#ifndef B200Q_H
#define B200Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t b200q_status;

/* Error vocabulary mirrors InferenceError (inference/crates/icn-contracts/src/lib.rs:709-723)
 * plus TIMEOUT for bounded device/host waits. */
enum {
    B200Q_OK = 0,
    B200Q_ERR_INVALID_CONFIG = 1, /* bad type id, K not a block multiple, null pointer, bad shard */
    B200Q_ERR_BACKEND = 2,        /* CUDA / NCCL failure; text in b200q_last_error */
    B200Q_ERR_CANCELLED = 3,
    B200Q_ERR_OVERLOADED = 4,     /* out of device memory */
    B200Q_ERR_STOPPED = 5,        /* context already destroyed / poisoned by a device error */
    B200Q_ERR_CALLBACK = 6,
    B200Q_ERR_TIMEOUT = 7         /* a bounded wait ran out (host sync or device pipeline) */
};

/* ggml tensor type ids, the values GGUF files carry (gguf.rs:126 reads them as u32). */
enum {
    B200Q_TYPE_F32 = 0,
    B200Q_TYPE_Q4_0 = 2,
    B200Q_TYPE_Q8_0 = 8,
    B200Q_TYPE_Q4_K = 12,
    B200Q_TYPE_Q5_K = 13,
    B200Q_TYPE_Q6_K = 14,
    B200Q_TYPE_BF16 = 30,
    B200Q_TYPE_MXFP4 = 39   /* on the tensor-core GEMM route the block scales must lie in 2^-24 .. 2^11 (fp16 operands) */
};

/* How a weight is cut for tensor parallelism (the reference only names the modes:
 * SplitMode::Row / SplitMode::Tensor, icn-contracts/src/lib.rs:200-205). */
enum {
    B200Q_SPLIT_COLUMN = 0, /* split output rows N: QKV, gate, up; no exchange */
    B200Q_SPLIT_ROW = 1     /* split K at 256-weight superblocks: O, down; outputs are partial sums */
};

/* Which kernel family b200q_matmul picked (b200q_last_route). */
enum {
    B200Q_ROUTE_NONE = 0,
    B200Q_ROUTE_GEMV = 1,   /* M <= 2 (up to 4 on request): dp4a streaming kernel on 16-bit fixed-point activations, HBM-bound */
    B200Q_ROUTE_SKINNY = 2, /* 3 <= M <= 16: streaming kernel, exact integer weights x exact bf16 activations in
                               mma.sync with fp32 accumulation, HBM-bound */
    B200Q_ROUTE_GEMM = 3    /* larger M: tcgen05 / TMEM GEMM, weights dequantized to fp16 in shared memory,
                               activations converted to fp16, fp32 accumulation */
};

/* Per-context settings (b200q_ctx_set_option). */
enum {
    /* smallest M that takes the SKINNY route (2..17; 17 = never); smaller batches use the GEMV kernel.
     * Default 3. */
    B200Q_OPT_SKINNY_MIN_M = 1,
    /* limit, in milliseconds, of every bounded wait inside the kernels (default 2000).  The value is
     * held per GPU and process, not per context: it applies to every context on the device. */
    B200Q_OPT_WAIT_LIMIT_MS = 2,
    /* host deadline of b200q_tp_init in milliseconds (default 60000) */
    B200Q_OPT_TP_INIT_TIMEOUT_MS = 3
};

typedef struct b200q_ctx b200q_ctx;
typedef struct b200q_weight b200q_weight;

/* -- library ------------------------------------------------------------------------------ */

/* "major.minor.patch" of this library; never NULL. */
const char *b200q_version(void);

/* Bytes of a GGUF tensor of `type` with `n_elements` weights, or -1 when the type is unknown or
 * the count is not a block multiple.  Same rule as llama_cpp_2::gguf::tensor_storage_bytes used
 * at inference/crates/icn-models/src/gguf.rs:129. */
int64_t b200q_tensor_storage_bytes(int32_t type, int64_t n_elements);

/* The same rule from the tensor's shape, as the reference calls it (type, shape): dims[0] is the row
 * length and must be a multiple of the type's block; every ggml tensor type a GGUF file may carry is
 * known here, not only the three the kernels multiply.  -1 for an unknown type or a bad shape. */
int64_t b200q_tensor_storage_bytes_shape(int32_t type, int32_t n_dims, const int64_t *dims);

/* -- context -------------------------------------------------------------------------------- */

/* One context per GPU / executor thread.  Replaces LlamaBackend::init + model.new_context
 * (icn-engine/src/lib.rs:141, 990) for this path. */
b200q_status b200q_ctx_create(int32_t device, b200q_ctx **out);
/* Weights and plans of the context are not destroyed with it and may be destroyed after it (they
 * keep what they need for that); every other call on them needs the context alive. */
void b200q_ctx_destroy(b200q_ctx *ctx);

/* Changes a per-context setting (B200Q_OPT_*); B200Q_ERR_INVALID_CONFIG for an unknown option or a
 * value outside its range.  No counterpart in the reference, whose backend takes its settings as
 * LlamaContextParams at creation (icn-engine/src/lib.rs:990). */
b200q_status b200q_ctx_set_option(b200q_ctx *ctx, int32_t option, int64_t value);

/* Copies the last error text of this context (NUL-terminated, truncated to n). */
b200q_status b200q_last_error(const b200q_ctx *ctx, char *buf, size_t n);

/* Waits for `stream` with a host-side deadline.  Replaces LlamaContext::synchronize
 * (icn-engine/src/lib.rs:1601-1615 uses it after a failed decode).  Also reads the device
 * status word: a kernel whose bounded pipeline wait ran out reports B200Q_ERR_TIMEOUT here. */
b200q_status b200q_sync(b200q_ctx *ctx, void *stream, uint64_t timeout_ms);

/* Kernel family chosen by the last b200q_matmul* call on this context (B200Q_ROUTE_*), and
 * the number of kernels that call launched. */
b200q_status b200q_last_route(const b200q_ctx *ctx, int32_t *route, int32_t *launches);

/* -- weights -------------------------------------------------------------------------------- */

/* Uploads a GGUF tensor (packed_host = N rows of K/blk blocks, `bytes` must equal
 * b200q_tensor_storage_bytes(type, N*K)).  The device copy is re-laid-out for 16-byte aligned
 * streaming (same byte count up to per-row padding).  Replaces the weight placement done inside
 * LlamaModel::load_from_file (icn-engine/src/lib.rs:972). */
b200q_status b200q_weight_upload(b200q_ctx *ctx, int32_t type, int64_t N, int64_t K,
                                 const void *packed_host, size_t bytes, b200q_weight **out);

/* Uploads only this rank's shard of the full tensor.  COLUMN: rows [N*rank/world, N*(rank+1)/world)
 * rounded to `align_rows` (pass the head size in rows for QKV, 0 or 1 otherwise).  ROW: superblock
 * columns [B*rank/world, B*(rank+1)/world) of every row, B = K/256 (remainders go to the low ranks,
 * e.g. 100 superblocks over 8 ranks = 13,13,13,13,12,12,12,12).  Replaces with_split_mode /
 * with_tensor_split (icn-hardware/src/lib.rs:2578-2589). */
b200q_status b200q_weight_upload_shard(b200q_ctx *ctx, int32_t type, int64_t N, int64_t K,
                                       const void *packed_host, size_t bytes, int32_t split,
                                       int32_t rank, int32_t world, int64_t align_rows,
                                       b200q_weight **out);

/* The range a rank owns under the rule above: rows for COLUMN, weights (multiples of 256; of 32
 * for Q8_0) for ROW.  Pure host arithmetic, usable without a device. */
b200q_status b200q_shard_range(int32_t type, int64_t N, int64_t K, int32_t split, int32_t rank,
                               int32_t world, int64_t align_rows, int64_t *begin, int64_t *end);

/* Host-only helpers (no device needed): the size of, and the conversion to, the device
 * ("streaming") layout of rows [0, N) of a GGUF tensor.  b200q_weight_upload applies the same
 * conversion; callers that cache converted weights on disk can use these directly.  The layout
 * pads N to a multiple of 4 rows: out_bytes = ((N + 3) / 4 * 4) * b200q_layout_row_bytes(type, K). */
int64_t b200q_layout_row_bytes(int32_t type, int64_t K);
b200q_status b200q_layout_pack(int32_t type, int64_t N, int64_t K, const void *packed_host,
                               size_t bytes, void *out_host, size_t out_bytes);

/* A second, independent device copy of a weight (distinct HBM addresses). */
b200q_status b200q_weight_clone(b200q_ctx *ctx, const b200q_weight *w, b200q_weight **out);

b200q_status b200q_weight_info(const b200q_weight *w, int32_t *type, int64_t *N, int64_t *K,
                               size_t *gguf_bytes, size_t *device_bytes);
void b200q_weight_destroy(b200q_weight *w);

/* Writes the N*K fp32 values the blocks encode to out_dev (row-major, device memory).
 * Bit-exact: fp16 scales widen exactly, each product/difference is one rounded fp32 operation,
 * no fused multiply-add.  (Qualified upstream by the dependency's test-quantize-fns,
 * inference/parity/upstream/targets.toml:38.) */
b200q_status b200q_dequantize(b200q_ctx *ctx, const b200q_weight *w, float *out_dev, void *stream);

/* The format's reference quantizer: N rows of K fp32 weights -> packed blocks in GGUF order
 * (out_bytes must equal b200q_tensor_storage_bytes(type, N * K)).  Host code, `threads` <= 0 = all
 * cores.  This is the encoder a model converter runs upstream of LlamaModel::load_from_file
 * (icn-engine/src/lib.rs:972); here it makes synthetic tensors for tests and benchmarks
 * ("quantized with the reference quantizer") without a model file. */
b200q_status b200q_quantize(int32_t type, const float *weights, int64_t N, int64_t K, void *packed_out, size_t out_bytes,
                            int32_t threads);

/* -- GGUF files ----------------------------------------------------------------------------- */

/* A parsed GGUF header: metadata keys and the tensor table.  Mirrors the bounded walk of the
 * reference's inspector (inference/crates/icn-models/src/gguf.rs:75-149): magic, version 2..3,
 * counts within the same bounds, every metadata value type, per tensor name / dimensions / type /
 * offset with overflow checks, alignment from general.alignment (default 32, power of two), header
 * rounded up to the alignment and inside the file.  No GPU is needed until b200q_gguf_upload. */
typedef struct b200q_gguf b200q_gguf;

typedef struct b200q_gguf_summary_t {
    uint32_t version;
    uint32_t alignment;
    uint64_t tensor_count;
    uint64_t metadata_count;
    uint64_t tensor_storage_bytes; /* sum over tensors, the figure of GgufInspection::tensor_storage_bytes (gguf.rs:34-35) */
    uint64_t header_bytes;         /* where the tensor data starts (gguf.rs:138-149) */
    uint64_t parameter_count;      /* general.parameter_count, else the sum of the tensors' elements */
    uint64_t file_bytes;
} b200q_gguf_summary_t;

typedef struct b200q_gguf_tensor_t {
    const char *name;     /* owned by the handle */
    uint32_t type;        /* ggml tensor type id */
    uint32_t n_dims;
    uint64_t dims[8];     /* dims[0] = row length K, dims[1] = rows N; unused entries are 1 */
    uint64_t elements;
    uint64_t bytes;
    uint64_t file_offset; /* absolute position of the tensor's data in the file */
} b200q_gguf_tensor_t;

/* Opens and parses `path`.  On failure *out is NULL and `err` (if given) holds the reason in the
 * reference's words ("file is not GGUF", "unsupported GGUF version 7", "GGUF header is
 * structurally invalid: ..."); B200Q_ERR_BACKEND for I/O errors, B200Q_ERR_INVALID_CONFIG for a
 * malformed file. */
b200q_status b200q_gguf_open(const char *path, b200q_gguf **out, char *err, size_t err_n);
void b200q_gguf_close(b200q_gguf *g);
b200q_status b200q_gguf_last_error(const b200q_gguf *g, char *buf, size_t n);
b200q_status b200q_gguf_summary(const b200q_gguf *g, b200q_gguf_summary_t *out);
/* A string-valued metadata key (e.g. "general.architecture"), or NULL; owned by the handle. */
const char *b200q_gguf_metadata_string(const b200q_gguf *g, const char *key);
/* An unsigned-integer-valued key with the reference's widening rules (gguf.rs:297-316). */
b200q_status b200q_gguf_metadata_u64(const b200q_gguf *g, const char *key, uint64_t *out);
b200q_status b200q_gguf_tensor_info(const b200q_gguf *g, uint64_t index, b200q_gguf_tensor_t *out);
b200q_status b200q_gguf_find(const b200q_gguf *g, const char *name, uint64_t *index);
/* Copies the tensor's packed bytes into dst (dst_bytes must equal its byte count). */
b200q_status b200q_gguf_read_tensor(b200q_gguf *g, uint64_t index, void *dst, size_t dst_bytes);
/* Reads tensor `index` (a Q8_0 / Q4_K / Q6_K matrix) and uploads it, whole (world = 1) or as the
 * shard of `rank` under the rule of b200q_weight_upload_shard.  Replaces, for one tensor, what
 * LlamaModel::load_from_file does for the whole file (icn-engine/src/lib.rs:972). */
b200q_status b200q_gguf_upload(b200q_ctx *ctx, b200q_gguf *g, uint64_t index, int32_t split, int32_t rank, int32_t world,
                               int64_t align_rows, b200q_weight **out);

/* -- the projection -------------------------------------------------------------------------- */

/* Y[M][N] = X[M][K] . W[N][K]^T   (ggml MUL_MAT with quantized src0; the op named at
 * inference/parity/cases/performance/backend-ops/native-perf-qualification.json:22).
 * x_dtype in {B200Q_TYPE_BF16, B200Q_TYPE_F32}; y_dtype in {B200Q_TYPE_F32, B200Q_TYPE_BF16}.
 * x_dev / y_dev are device pointers; ldx >= K, ldy >= N.  M == 0 is a no-op.
 * The kernel family is chosen by M (see B200Q_ROUTE_*). */
b200q_status b200q_matmul(b200q_ctx *ctx, const b200q_weight *w, const void *x_dev, int32_t x_dtype,
                          int64_t M, int64_t ldx, void *y_dev, int32_t y_dtype, int64_t ldy,
                          void *stream);

/* Several weights of the same type and K applied to one activation in a single launch
 * (gate+up, or Q+K sharing x): Y_i[M][N_i] = X . W_i^T.  n_weights <= 4.  Falls back to one
 * launch per weight for M > 4. */
b200q_status b200q_matmul_multi(b200q_ctx *ctx, const b200q_weight *const *w, int32_t n_weights,
                                const void *x_dev, int32_t x_dtype, int64_t M, int64_t ldx,
                                void *const *y_dev, int32_t y_dtype, const int64_t *ldy, void *stream);

/* The same product with HOST activations and outputs: copies X to the device, runs the
 * projection, copies Y back and waits — the shape of the reference's own boundary, where
 * decode() takes host tokens and get_logits_ith returns host floats
 * (icn-engine/src/lib.rs:2264, parity_probe.rs:701). */
b200q_status b200q_matmul_host(b200q_ctx *ctx, const b200q_weight *w, const void *x_host,
                               int32_t x_dtype, int64_t M, int64_t ldx, void *y_host,
                               int32_t y_dtype, int64_t ldy);

/* Host-buffer form of b200q_matmul_multi. */
b200q_status b200q_matmul_multi_host(b200q_ctx *ctx, const b200q_weight *const *w, int32_t n_weights,
                                     const void *x_host, int32_t x_dtype, int64_t M, int64_t ldx,
                                     void *const *y_host, int32_t y_dtype, const int64_t *ldy);

/* The prefill product for callers that must not allocate device memory.  No counterpart in the
 * reference: there the engine sizes a model's whole GPU footprint before loading it and keeps the
 * device to that plan, so a library that quietly grows a scratch buffer with cudaMalloc in the
 * middle of serving can fail, or push the process past the budget it was admitted under; a host
 * that has handed every free byte to its own pool has nothing left to give at all.  This entry
 * point keeps the 16-bit copy of the activations in a fixed 8 MiB array inside the library image
 * instead (each GPU that loads the library holds it until the process exits) and calls no
 * allocator.  It always takes the tensor-core route.
 *   - limit: M * round_up(K, 8) <= 4,194,304 elements; larger requests fail with
 *     B200Q_ERR_INVALID_CONFIG and a message naming both numbers;
 *   - the first call on a device looks up the array's device address; make that call before any
 *     stream capture is begun;
 *   - all calls on a device share the array: calls whose GPU work can overlap (different streams)
 *     race on it, so keep them on one stream or order them yourself. */
b200q_status b200q_matmul_prefill_noalloc(b200q_ctx *ctx, const b200q_weight *w, const void *x_dev,
                                          int32_t x_dtype, int64_t M, int64_t ldx, void *y_dev,
                                          int32_t y_dtype, int64_t ldy, void *stream);

/* -- decode plans ------------------------------------------------------------------------------ */

/* A plan is a fixed list of projections (1..16 activation rows, the same M for all) prepared once
 * and run many times.  With 1..2 rows (the route edge B200Q_OPT_SKINNY_MIN_M moves it up to 4 rows;
 * plans with rank sums, SWIGLU, ACCUMULATE or fused-norm jobs always, and with at most 4 rows) one
 * launch executes the jobs back to back on persistent CTAs: the weights of projection i+1 stream
 * from HBM while projection i is still being reduced and stored, so a decode step is not broken up
 * by launch gaps.  With more rows (a verify batch) consecutive jobs of one block type run as
 * skinny-kernel launches of up to 32 products each.  It plays the role of the per-token graph that context.decode(batch) runs for a
 * batch of 1..4 tokens (inference/crates/icn-engine/src/lib.rs:2264).  Pointers are captured at
 * creation: run the plan again after rewriting the activation buffers in place. */
typedef struct b200q_plan b200q_plan;

enum {
    /* the job's activation is written by earlier jobs of the same plan (e.g. the down projection
     * reading what gate/up produced): all CTAs finish those jobs before this one converts x */
    B200Q_JOB_WAITS_FOR_EARLIER = 1,
    /* row-parallel projection under tensor parallelism: the job's outputs are partial sums, and the
     * launch itself adds them up over the ranks attached with b200q_peer_attach (peer-memory stores
     * and loads from inside the kernel, no separate all-reduce).  One weight, fp32 output, M x N at
     * most B200Q_PEER_MAX_COUNT; every rank must run the same plan.  Without attached peers the
     * flag does nothing (the sum over one rank is the output itself). */
    B200Q_JOB_SUM_RANKS = 2,
    /* gated MLP: the job has exactly two weights of equal shape, w[0] = gate and w[1] = up, and writes
     * y_dev[0][m][n] = silu(gate x)[n] * (up x)[n] (silu(v) = v / (1 + exp(-v)), in fp32); y_dev[1] is not
     * used.  The activation function llama-style models apply between the two projections and `down`
     * (the reference runs it as a separate ggml op of the same graph).  Streaming plans only (M <= 4). */
    B200Q_JOB_SWIGLU = 4,
    /* residual connection: the job adds its result to what y_dev holds instead of overwriting it; with
     * B200Q_JOB_SUM_RANKS the sum over the ranks is added once, on every rank.  Streaming plans only. */
    B200Q_JOB_ACCUMULATE = 8
};

typedef struct b200q_job {
    const b200q_weight *w[4]; /* 1..4 weights of one type and K sharing x */
    int32_t n_weights;
    int32_t x_dtype;          /* B200Q_TYPE_BF16 or B200Q_TYPE_F32 */
    const void *x_dev;        /* X[M][K], device memory */
    int64_t ldx;
    void *y_dev[4];           /* Y_i[M][N_i], device memory */
    int64_t ldy[4];
    int32_t y_dtype;          /* B200Q_TYPE_F32 or B200Q_TYPE_BF16 */
    int32_t flags;            /* B200Q_JOB_* */
    /* RMSNorm fused into the activation load: when norm_weight is not NULL the job multiplies
     * x_norm[m][k] = x[m][k] * rsqrt(mean_k(x[m][k]^2) + norm_eps) * norm_weight[k] (fp32 arithmetic;
     * norm_weight = K floats in device memory) instead of x: the normalisation llama-style models
     * apply before QKV and before gate/up.  Streaming plans only (M <= 4). */
    const float *norm_weight;
    float norm_eps;
    int32_t reserved;         /* 0: zero-initialise the struct; a non-zero value is refused (it catches uninitialised jobs) */
} b200q_job;

b200q_status b200q_plan_create(b200q_ctx *ctx, const b200q_job *jobs, int32_t n_jobs, int64_t M,
                               b200q_plan **out);
b200q_status b200q_plan_run(b200q_ctx *ctx, b200q_plan *plan, void *stream);
void b200q_plan_destroy(b200q_plan *plan);

/* -- tensor parallel exchange ------------------------------------------------------------------ */

/* 128-byte NCCL unique id for rank 0 to broadcast out of band. */
b200q_status b200q_tp_unique_id(void *id_out_128);

/* Joins a `world`-rank NCCL communicator on this context's device.  The reference has no
 * collective of its own (its multi-GPU is llama.cpp's in-process split); this is the single
 * all-reduce a row-parallel projection (O, down) needs.  Gives up with B200Q_ERR_TIMEOUT after
 * B200Q_OPT_TP_INIT_TIMEOUT_MS when some rank never joins.  While a communicator is attached,
 * b200q_sync also asks NCCL for asynchronous errors and aborts the communicator when one is
 * reported or when its own deadline passes, so a collective that a failed rank never enters does
 * not hold the stream for ever. */
b200q_status b200q_tp_init(b200q_ctx *ctx, int32_t rank, int32_t world, const void *id_128);

/* In-place sum over ranks of y_dev[count] (dtype F32 or BF16) on `stream`. */
b200q_status b200q_allreduce(b200q_ctx *ctx, void *y_dev, int64_t count, int32_t dtype, void *stream);

b200q_status b200q_tp_finalize(b200q_ctx *ctx);

/* Low-latency exchange for decode-sized vectors: ranks that are processes on one NVLink-connected
 * node map each other's exchange buffer (CUDA IPC) and b200q_allreduce then sums fp32 vectors of up
 * to B200Q_PEER_MAX_COUNT elements with one kernel of peer stores and loads instead of NCCL.
 *   1. every rank: b200q_peer_export -> a 64-byte handle of its own buffer;
 *   2. the caller gathers the handles of all ranks (rank order) out of band;
 *   3. every rank: b200q_peer_attach(rank, world <= 8, handles).
 * All ranks must then issue the same sequence of b200q_allreduce calls.  No reference counterpart
 * (see b200q_tp_init). */
#define B200Q_PEER_HANDLE_BYTES 64
#define B200Q_PEER_MAX_COUNT 16384
b200q_status b200q_peer_export(b200q_ctx *ctx, void *handle_out_64);
b200q_status b200q_peer_attach(b200q_ctx *ctx, int32_t rank, int32_t world, const void *handles);
b200q_status b200q_peer_detach(b200q_ctx *ctx);

/* The same exchange for ONE process that drives several GPUs (or several contexts) itself: the
 * exchange buffers are passed as device pointers instead of IPC handles.
 *   1. every context: b200q_peer_buffer -> its own buffer;
 *   2. the caller enables peer access between the devices (cudaDeviceEnablePeerAccess);
 *   3. every context: b200q_peer_attach_buffers(rank, world, buffers) with buffers[rank] its own.
 * After B200Q_ERR_TIMEOUT from an exchange the ranks' call counters may disagree: further exchanges
 * fail with B200Q_ERR_STOPPED until every rank has detached and attached again (both forms). */
b200q_status b200q_peer_buffer(b200q_ctx *ctx, void **buffer_out);
b200q_status b200q_peer_attach_buffers(b200q_ctx *ctx, int32_t rank, int32_t world, void *const *buffers);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
