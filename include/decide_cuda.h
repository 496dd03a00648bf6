/* decide_cuda.h — C ABI of libdecide_cuda.so, the sm_100a (B200) backend behind decide's
 * operator interface.
 *
 * It replaces the reference's `decide-metal` device layer and `kernels/*.metal` behind the
 * `decide-engine` dispatch wrappers (crates/decide-engine/src/kernels/mod.rs:40-67): one
 * entry point per wrapper method, same argument meaning.
 *
 * Conventions (they mirror the reference's, kernels/mod.rs:1-5 and 31-38):
 *  - Every dc_<op> only ENQUEUES work on `stream` (a cudaStream_t passed as void*) and
 *    returns; it never synchronises. Stream order is the only ordering, as the serial
 *    compute encoder is in the reference (forward.rs:31-38).
 *  - Pointers are device pointers already offset to the first element (the reference passes
 *    (buffer, byte offset) pairs). Dims and strides are in ELEMENTS, enums are uint32_t.
 *  - The caller owns every buffer. The context owns only its tensor-map cache, a status
 *    word and a bounded scratch workspace.
 *  - Return value 0 = DC_OK. Contract violations that the reference `assert!`s return
 *    DC_INVALID_ARG with a message readable through dc_last_error (latched, cleared on
 *    read), in the style of the reference's own C ABI (crates/decide-ane/src/lib.rs:22-35).
 *  - There is no CPU fallback: without a CUDA device dc_open fails.
 *  - A context is not thread-safe (the reference's Forward::logits takes &mut self,
 *    forward.rs:704) and serves ONE stream at a time: its scratch workspace, the partial-sum
 *    buffers of the split GEMM and their arrival counters are one per context, so two streams
 *    running ops of one context concurrently race on them. Distinct contexts are independent.
 *  - Ops that need scratch (dc_attention with seq_start, dc_gated_delta, dc_conv_gated_delta,
 *    dc_convert_bf16_to_f16) take it from the context's workspace. If the workspace is too small
 *    the op grows it: a cudaFree + cudaMalloc, i.e. a device-wide synchronisation inside the
 *    call, which also fails under stream capture. To keep requests allocation-free, call
 *    dc_reserve_workspace once with the largest demand (dc_gated_delta_scratch_bytes,
 *    dc_attention_scratch_bytes), then dc_set_workspace_frozen(ctx, 1): from then on an op that
 *    would have grown the workspace returns DC_INVALID_ARG instead. dc_model_* does both itself.
 */
#ifndef DECIDE_CUDA_H
#define DECIDE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dc_ctx dc_ctx;

enum {
    DC_OK = 0,
    DC_INVALID_ARG = 1,   /* what the reference asserts on */
    DC_CUDA_ERROR = 2,    /* a CUDA call failed */
    DC_UNSUPPORTED = 3,   /* shape/feature outside what the kernels are built for */
    DC_TIMEOUT = 4        /* a bounded device-side wait ran out (see dc_check_status) */
};

/* Epilogue of dc_gemm: kernels/gemm.rs:16-26 (fp16 there, bf16 here). */
enum {
    DC_EPI_STORE_F32 = 0,   /* Y fp32 [M,N] = acc */
    DC_EPI_STORE_BF16 = 1,  /* Y bf16 [M,N] = acc */
    DC_EPI_ADD_F32 = 2,     /* Y fp32 [M,N] += acc (the residual add) */
    DC_EPI_SWIGLU_BF16 = 3  /* Y bf16 [M,N/2] = silu(gate)*up over interleaved gate|up blocks */
};

/* Kernel choice per family, the reference's DECIDE_GEMM / DECIDE_ATTN / DECIDE_DELTA = fast|baseline
 * (kernels/gemm.rs:56-63, attn.rs:49-56, delta.rs:34-41). */
enum { DC_IMPL_FAST = 0, DC_IMPL_BASELINE = 1 };
enum { DC_FAMILY_GEMM = 0, DC_FAMILY_ATTN = 1, DC_FAMILY_DELTA = 2 };

/* The 16-bit type of a context: every 16-bit GEMM operand, i.e. the activations (normed rows, gated
 * outputs, the MLP intermediate, attention q/k/v and its output) AND the weight matrices, is stored
 * in it. The embedding table is always bf16. The reference converts its bf16 checkpoint to fp16 and
 * keeps fp16 activations because bf16 missed its 0.01 probability tolerance (README.md:88-90,
 * 207-208; convert.rs:73-90); DC_ACT_F16 is the default here for the same measured reason (bf16
 * activations alone put ~0.6% relative error into the residual per layer). dc_convert_bf16_to_f16
 * converts bf16 weights. Wherever this header says "bf16" for a GEMM operand or an activation
 * buffer, read "the context's 16-bit type". The tensor cores cannot mix the two in one MMA. */
enum { DC_ACT_BF16 = 0, DC_ACT_F16 = 1 };
/* Tensor-core engines of the fast attention and delta-rule kernels: see dc_set_engine. */
enum { DC_ENGINE_MMA_SYNC = 0, DC_ENGINE_TCGEN05 = 1 };

/* ---- context: replaces DecideDevice::shared + Kernels::new (device.rs:125-130, mod.rs:54-66) ---- */
dc_ctx* dc_open(int device, char* err, size_t err_len);
void dc_close(dc_ctx* ctx);
/* Copies the latched error message (empty when none) and clears it; returns its length. */
size_t dc_last_error(dc_ctx* ctx, char* buf, size_t len);
/* Picks fast or baseline kernels for a family; at open the DECIDE_GEMM / DECIDE_ATTN /
 * DECIDE_DELTA environment variables are read once, as Gemm::new etc. do. */
int dc_set_impl(dc_ctx* ctx, uint32_t family, uint32_t impl);
uint32_t dc_get_impl(dc_ctx* ctx, uint32_t family);
/* The context's 16-bit type (DC_ACT_*); at open it is read from DECIDE_ACT = f16 | bf16 (default f16). */
int dc_set_activation_dtype(dc_ctx* ctx, uint32_t act);
uint32_t dc_get_activation_dtype(dc_ctx* ctx);
/* Operand precision of the chunked gated delta rule's tensor-core products: 3 (default; also
 * DECIDE_DELTA_SPLIT=3) takes every fp32 operand as hi + lo bf16 parts, 3 MMAs per product, ~1e-5
 * relative error against fp32; 1 is a single bf16 pass, 3x fewer MMAs, ~3e-3 relative error in o. */
int dc_set_delta_split(dc_ctx* ctx, uint32_t split);
/* Tensor-core engine of a family's FAST kernels: DC_ENGINE_TCGEN05 (default) or DC_ENGINE_MMA_SYNC, the
 * register-accumulator forms on mma.sync. At open: DECIDE_ATTN_ENGINE / DECIDE_DELTA_ENGINE = tcgen05 | mma.
 *  DC_FAMILY_DELTA: the serial kernel of the chunked delta rule with split 3 (split 1 always runs on
 *    mma.sync); tcgen05 keeps the accumulators in tensor memory, one CTA per (sequence, head); mma.sync
 *    also splits the value columns over CTAs. Same results to ~1e-6.
 *  DC_FAMILY_ATTN: tcgen05 serves packed batches (seq_start given) and chunks of one sequence whose cache
 *    length is given (dc_attention); other calls without seq_start run on mma.sync. Same contract;
 *    results differ by fp32 rounding order only.
 *  DC_FAMILY_GEMM has one engine (tcgen05). */
int dc_set_engine(dc_ctx* ctx, uint32_t family, uint32_t engine);
/* Synchronises `stream`, then reports DC_TIMEOUT if a kernel's bounded wait ran out since the
 * last check (the analogue of the command-buffer status check, forward.rs:1022-1042), or
 * DC_INVALID_ARG if a kernel found a contract violation only it can see (dc_attention: a position at
 * or past the cache length given). */
int dc_check_status(dc_ctx* ctx, void* stream);
/* Self-test of that path (no counterpart in the reference): enqueues one tiny kernel whose only
 * wait is on an mbarrier that nothing ever arrives at. The wait gives up at the library's limit
 * (400 ms), raises the status word with wait id 99 and the kernel returns normally; the next
 * dc_check_status must report DC_TIMEOUT and the context stays usable. */
int dc_selftest_wait_timeout(dc_ctx* ctx, void* stream);
/* Kernels enqueued through this context so far. */
uint64_t dc_launch_count(dc_ctx* ctx);
/* Grows the context's scratch workspace to at least `bytes` now, so that later calls do not
 * allocate (Gemm::warm_up's role for pipelines, gemm.rs:89-107). */
int dc_reserve_workspace(dc_ctx* ctx, size_t bytes);
/* on = 1: an op that needs more scratch than is reserved returns DC_INVALID_ARG (naming the demand)
 * instead of freeing and reallocating the workspace; on = 0 restores growing on demand. */
int dc_set_workspace_frozen(dc_ctx* ctx, uint32_t on);
size_t dc_workspace_bytes(dc_ctx* ctx);
/* Makes every kernel variant launchable now (opts each into its shared-memory size on this device), so
 * that no request does it: Gemm::warm_up (kernels/gemm.rs:89-107; checked in engine.rs:168-172).
 * dc_model_create calls it. */
int dc_warm_up(dc_ctx* ctx);
/* What the "nothing is allocated or encoded inside a request" rule can be checked with
 * (device.rs:482-543 keeps the same kind of cache for pipelines): device/pinned allocations this
 * context has made so far (open, workspace growth, dc_model_create), tensor maps encoded so far
 * (cache misses), and the number of cached tensor maps. A second request of a shape the context has
 * already served leaves all three unchanged. The cache is dropped whole when it reaches 8,192 maps. */
uint64_t dc_alloc_count(dc_ctx* ctx);
uint64_t dc_tmap_encode_count(dc_ctx* ctx);
size_t dc_tmap_cache_size(dc_ctx* ctx);
/* Number of SMs of the context's device. */
int dc_sm_count(dc_ctx* ctx);
/* Content hash (16 hex digits) of the kernel sources this library was built from: the stale-binary guard of
 * the reference (crates/decide-metal/src/source_hash.rs:47-62; lib.rs:18-21). A host that ships the sources
 * beside the library compares it with the hash of those sources before use, as the Python binding does. */
const char* dc_source_hash(void);

/* ---- weight conversion (bf16_to_f16 of the converter, crates/decide-engine/src/convert.rs:73-90) ----
 * dst[i] = fp16(src[i]) for n bf16 values, round to nearest even; dst may be src (in place). Adds to
 * *report (host memory, may be NULL) how many values became fp16 subnormals, were flushed to zero or
 * overflowed to infinity, as the reference's precision-loss report does. Synchronises the stream. */
typedef struct dc_convert_report {
    uint64_t values, f16_subnormal, f16_flushed_to_zero, f16_overflow;
} dc_convert_report;
int dc_convert_bf16_to_f16(dc_ctx* ctx, void* stream, const void* src, void* dst, size_t n, dc_convert_report* report);

/* ---- the same conversion for callers that must not allocate ----
 * No counterpart in the reference. It exists for hosts that swap a checkpoint in while another
 * stream is serving requests, or that have already handed all device memory to one arena: for them
 * cudaMalloc is off the table (it stalls every stream of the device while it runs, and it can simply
 * fail when the arena owns the memory), and dc_open / dc_convert_bf16_to_f16 both allocate (the
 * status word, the workspace holding the counters). This entry point needs no context and calls no
 * cudaMalloc, cudaFree or other allocating routine: its four 64-bit counters live in a static array
 * inside the library image, 256-byte aligned, which every GPU that loads the library holds until the
 * process exits. It works on the CURRENT device and `stream` must belong to it.
 *  - Limit: at most DC_NOALLOC_MAX_VALUES (2^32) values per call; larger n is refused with
 *    DC_INVALID_ARG and a message in `err` (split the tensor).
 *  - The first call on each device looks the array's device address up (cudaGetSymbolAddress);
 *    make that first call before any stream capture begins on that device. With CUDA's lazy
 *    module loading that first look-up and launch also make the driver load this library's
 *    kernel image onto the device, which takes device memory: the guarantee "nothing is
 *    allocated" holds from the SECOND call on a device onwards, so warm the entry point up (an
 *    n = 0 call is enough) before the no-allocation regime starts. First calls on one device
 *    may come from several threads at once (the look-up is idempotent and stored atomically).
 *  - All calls share the one array, which still holds the previous call's counts: it is cleared on
 *    `stream` at the start of every call. Two calls that overlap on the GPU (different streams, or
 *    host threads racing on one device) corrupt each other's report; serialise them.
 * Otherwise as dc_convert_bf16_to_f16: dst may be src, *report (may be NULL) is added to, the stream
 * is synchronised before returning. `err` (may be NULL) receives the message of a failure. */
#define DC_NOALLOC_MAX_VALUES (1ull << 32)
int dc_convert_bf16_to_f16_noalloc(void* stream, const void* src, void* dst, size_t n, dc_convert_report* report,
                                   char* err, size_t err_len);

/* ---- Gemm::gemm (kernels/gemm.rs:138-175; spec cpu_ref.rs:25-50) ----
 * Y = X * W^T then `epilogue`. X bf16 [M,K] row stride ldx; W bf16 [N,K] row stride ldw;
 * ldy in elements of Y's type. fp32 accumulation. Requires N%32==0, K%32==0, M>=1,
 * ldx,ldw >= K, ldy >= output columns. The fast (tcgen05) kernels also need ldx%8==0, ldw%8==0,
 * x,w 16-byte aligned, ldy%8==0 (bf16 outputs) or ldy%4==0 (fp32 outputs), y 16-byte aligned, and
 * swiglu_block == 16 for DC_EPI_SWIGLU_BF16 (as gemm_fast.metal hard-codes).
 * M <= DC_GEMM_SMALL_MAX_M runs the weight-streaming small-M kernel (the reference's gemm_nt_small,
 * kernels/gemm_fast.metal:470-517, chosen for M <= 16 by gemm_configs.rs:252-267); larger M the tcgen05
 * kernel. dc_gemm_tile always runs the tcgen05 kernel, whatever M. */
#define DC_GEMM_SMALL_MAX_M 16u
int dc_gemm(dc_ctx* ctx, void* stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k,
            uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epilogue, uint32_t swiglu_block);

/* Test hooks for the fast GEMM: dc_gemm_tile forces the output tile width (128, 192, 224 or 256) that
 * the plan would otherwise choose per shape (the role of gemm_configs::plan,
 * crates/decide-metal/src/gemm_configs.rs:312, and of the reference's per-config test sweep).
 * DECIDE_GEMM_BN = 128 | 192 | 224 | 256 forces it for every dc_gemm of the process, DECIDE_GEMM_SPLIT = 1..4
 * caps the K split of the tail wave. */
int dc_gemm_tile(dc_ctx* ctx, void* stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k,
                 uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epilogue, uint32_t bn);
/* The plan for a shape and epilogue: returns the tile width (bn = 0: the planner's choice; otherwise the plan
 * dc_gemm_tile follows for that width; 0 is returned for a width the kernel does not have) and stores into
 * *tail_split (may be NULL) the number of parts each tile of the last, partial wave is cut into along K
 * (1 = whole tiles). With an fp32 output the parts accumulate into Y in part order; with a 16-bit output they
 * meet in the context's workspace. Either way the result does not depend on timing. */
uint32_t dc_gemm_plan_for(dc_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t epilogue, uint32_t bn, uint32_t* tail_split);
/* Shorthands: the tile width for K = 2560 and an fp32 store; width and split for a given K and the `+=` epilogue. */
uint32_t dc_gemm_plan(dc_ctx* ctx, uint32_t m, uint32_t n);
uint32_t dc_gemm_plan_k(dc_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t* tail_split);

/* ---- Norm::rmsnorm (kernels/norm.rs:23-33; spec cpu_ref.rs:11-22) ----
 * y[r] = x[rowmap[r]] * rsqrt(mean(x^2)+eps) * (add_one ? 1+w : w); x fp32, w fp32 [h], y bf16.
 * rowmap u32 [rows] or NULL for the identity. h%4==0. */
int dc_rmsnorm(dc_ctx* ctx, void* stream, const float* x, const float* w, void* y, const uint32_t* rowmap,
               uint32_t rows, uint32_t h, uint32_t ld_in, uint32_t ld_out, float eps, uint32_t add_one);

/* ---- Ane::add_partial + Norm::rmsnorm in one pass (kernels/ane.rs:23, kernels/ane.metal:10-18; norm.rs:23-33) ----
 * x[r] += add[r] over `rows` dense fp32 rows of h values (the summed partial outputs of a row-split
 * projection join the residual), then, unless y is NULL, y[r] = rmsnorm(x[r]) as dc_rmsnorm writes it. */
int dc_add_rmsnorm(dc_ctx* ctx, void* stream, float* x, const float* add, const float* w, void* y, uint32_t rows, uint32_t h,
                   float eps, uint32_t add_one);
/* The same with `add16` in the context's 16-bit type (partial sums exchanged in 16 bits, dc_tp_set_exchange_16bit). */
int dc_add16_rmsnorm(dc_ctx* ctx, void* stream, float* x, const void* add16, const float* w, void* y, uint32_t rows, uint32_t h,
                     float eps, uint32_t add_one);

/* ---- tensor-parallel group (no counterpart in the reference beyond its two-way GPU + Neural Engine MLP
 * split with a partial-sum add, forward.rs:270-303, 1286-1309) ----
 * One process and one context per GPU. dc_tp_unique_id makes a 128-byte id on one rank; the host hands
 * it to every rank; dc_tp_init (collective: every rank calls it) joins the context to the group, NCCL
 * being loaded with dlopen at that moment (DECIDE_NCCL_LIB names the library if it is not on the
 * loader's path). A dc_model created on a context that is in a group of G > 1 is one RANK's SHARD: its
 * dc_dims carry the rank's head counts and intermediate size (nq/G, nkv/G, gdn_nk/G, gdn_nv/G, inter/G,
 * hidden whole), its weights are the matching slices (in-projections and gate_up by output row, out and
 * down projections by input column), and its forward all-reduces the fp32 [rows, hidden] partial sums
 * after each row-split projection. Embedding, norms, residual and head are replicated.
 * dc_tp_all_reduce_f32 is that exchange (in place, enqueued on `stream`). */
int dc_tp_unique_id(void* id128, char* err, size_t err_len);
int dc_tp_init(dc_ctx* ctx, const void* id128, uint32_t world, uint32_t rank);
int dc_tp_all_reduce_f32(dc_ctx* ctx, void* stream, float* buf, size_t n);
/* The exchange in the context's 16-bit type: n values of `buf` summed over the group in place (NCCL adds them in that
 * type). dc_tp_set_exchange_16bit(ctx, 1), or DECIDE_TP_EXCHANGE=16 at dc_tp_init, makes a shard's forward store its
 * partial sums in 16 bits, exchange half the bytes and widen them when they join the fp32 residual; default fp32. */
int dc_tp_all_reduce_16(dc_ctx* ctx, void* stream, void* buf, size_t n);
int dc_tp_set_exchange_16bit(dc_ctx* ctx, uint32_t on);
uint32_t dc_tp_world(dc_ctx* ctx);
uint32_t dc_tp_rank(dc_ctx* ctx);
void dc_tp_destroy(dc_ctx* ctx);

/* ---- Embed::embed (kernels/embed.rs:16-22) ---- out[t] = float(table[ids[t]]), table bf16 [vocab,h]. */
int dc_embed(dc_ctx* ctx, void* stream, const uint32_t* ids, const void* table, float* out, uint32_t t, uint32_t h);

/* ---- Head::gather_rows_f32 / gather_rows_f16 (kernels/head.rs:28-45) ---- out[i] = x[rowmap[i]]. */
int dc_gather_rows_f32(dc_ctx* ctx, void* stream, const float* x, const uint32_t* rowmap, float* out, uint32_t rows,
                       uint32_t h);
int dc_gather_rows_bf16(dc_ctx* ctx, void* stream, const void* x, const uint32_t* rowmap, void* out, uint32_t rows,
                        uint32_t h);

/* ---- Head::final_head (kernels/head.rs:47-60; spec cpu_ref.rs:192-198) ----
 * Final zero-centred RMSNorm (weight w fp32 [h]) of each of `rows` fp32 rows of x [rows,h], then
 * logits against the bf16 rows of `table` named by cand (u32 [rows,max_cand], row r uses the first
 * ncand[r]). Writes fp32 logits [rows,max_cand]; entries past ncand[r] are not written. */
int dc_final_head(dc_ctx* ctx, void* stream, const float* x, const float* w, const void* table,
                  const uint32_t* cand, const uint32_t* ncand, float* logits, uint32_t rows, uint32_t h,
                  uint32_t max_cand, float eps);

/* ---- GNorm::gated_rmsnorm_silu (kernels/gnorm.rs:19-31; spec cpu_ref.rs:132-145) ----
 * Per (row, value head): RMSNorm of o (fp32 [t,nv,dv]) over dv with weight w (fp32 [dv], no +1),
 * times silu(z); z is read from rows of stride ldz (head h at columns h*dv..). Writes bf16 y [t,nv*dv].
 * dv must be 128. */
int dc_gated_rmsnorm_silu(dc_ctx* ctx, void* stream, const float* o, const float* z, const float* w, void* y,
                          uint32_t t, uint32_t nv, uint32_t dv, uint32_t ldz, float eps);

/* ---- Rope::q_norm_rope (kernels/rope.rs:26-37; spec cpu_ref.rs:149-162) ----
 * Zero-centred per-head RMSNorm (weight qw fp32 [hd]) + RoPE on the first `rot` dims (pairs i, i+rot/2,
 * fp32 angle = qpos[r] * inv_freq[i], precise sin/cos) of the nq q heads of `rows` rows of pq (fp32,
 * q at column 0, row stride ldq). Writes bf16 qo [rows,nq,hd]. hd 128 or 256; rot%8==0, rot<=128. */
int dc_q_norm_rope(dc_ctx* ctx, void* stream, const float* pq, const float* qw, const float* inv_freq,
                   const uint32_t* qpos, void* qo, uint32_t rows, uint32_t ldq, uint32_t nq, uint32_t hd,
                   uint32_t rot, float eps);

/* ---- Rope::kv_norm_rope (kernels/rope.rs:39-51) ----
 * For `rows` rows of pkv (fp32, row stride ldkv): norm+RoPE of the nkv k heads (at column kcol) into the K
 * cache kc and a copy of the nkv v heads (at column vcol) into the V cache vc, both bf16 [cache_rows,nkv,hd].
 * With pos == NULL row r is at position pos0 + r and is written to cache row pos0 + r (the reference's
 * form). With pos (u32 [rows], packed sequences) row r is rotated for position pos[r] and written to
 * cache row r. Rows past cache_rows are refused (rope.rs:45). */
int dc_kv_norm_rope(dc_ctx* ctx, void* stream, const float* pkv, const float* kw, const float* inv_freq, void* kc,
                    void* vc, uint32_t rows, uint32_t ldkv, uint32_t kcol, uint32_t vcol, uint32_t pos0,
                    const uint32_t* pos, uint32_t cache_rows, uint32_t nkv, uint32_t hd, uint32_t rot, float eps);

/* ---- Attn::attention (kernels/attn.rs:81-118; spec cpu_ref.rs:167-188) ----
 * Causal GQA attention: query row r (bf16 q [rows,nq,hd]) at position qpos[r] attends cache rows
 * 0..=qpos[r] of the bf16 K/V caches [..,nkv,hd]; scale hd^-1/2; fp32 online softmax. `gate` (fp32,
 * row stride ldg, already offset to the gate's first column; NULL = no gate) multiplies the output by
 * sigmoid(gate). Writes bf16 y [rows, nq*hd]. hd must be 128.
 * seq_start == NULL: one sequence; max_len, if not 0, is the number of cache rows in use (every
 * qpos[r] < max_len, the cache holds at least that many rows): a chunk of 64 or more rows that
 * continues a longer cache then runs on the tcgen05 kernel (rows past max_len are never read; a
 * position at or past max_len is reported by the next dc_check_status as DC_INVALID_ARG), with
 * max_len = 0 it runs on the mma.sync kernel. Otherwise seq_start is u32 [n_seq+1] row offsets of
 * packed sequences (q rows and cache rows packed alike, qpos relative to the sequence) and max_len
 * the longest sequence. */
int dc_attention(dc_ctx* ctx, void* stream, const void* q, const void* kc, const void* vc, const float* gate,
                 const uint32_t* qpos, void* y, uint32_t rows, uint32_t ldg, uint32_t nq, uint32_t nkv, uint32_t hd,
                 const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len);

/* ---- Attn::attention for answer rows of a packed batch (the call of the pruned last layer,
 * forward.rs:1176-1178: a few query rows at given positions over the whole cache) ----
 * As dc_attention without seq_start, plus kv_start (u32 [rows], NULL = all 0): query row r attends
 * cache rows kv_start[r] .. kv_start[r] + qpos[r], i.e. the cache rows of its own request in a
 * packed batch. Built for few rows: one CTA per (row, kv head, slice of the keys), fp32 throughout;
 * when rows * nkv would leave most SMs idle each row's keys are cut into slices whose partial sums go
 * through the context workspace (dc_attention_rows_scratch_bytes: reserve it before freezing the
 * workspace) and are joined in slice order. nq / nkv <= 16. */
int dc_attention_rows(dc_ctx* ctx, void* stream, const void* q, const void* kc, const void* vc, const float* gate,
                      const uint32_t* qpos, const uint32_t* kv_start, void* y, uint32_t rows, uint32_t ldg, uint32_t nq,
                      uint32_t nkv, uint32_t hd);
size_t dc_attention_rows_scratch_bytes(dc_ctx* ctx, uint32_t rows, uint32_t nq, uint32_t nkv);

/* ---- Conv::conv_silu_l2 (kernels/conv.rs:21-36; spec cpu_ref.rs:55-81) ----
 * Depthwise causal conv (kernel 4) + SiLU over the qkv columns 0..(2nk+nv)*128 of `t` rows of p (fp32,
 * row stride ldp); prev = the 3 raw rows before them (fp32 [3,conv_dim], oldest first; NULL = zeros);
 * w fp32 [conv_dim,4]. Writes fp32 q,k [t,nk,dk] (L2-normed, q also scaled by dk^-1/2) and v [t,nv,dv].
 * dk = dv = 128. Packed sequences: seq_start u32 [n_seq+1], prev [n_seq,3,conv_dim], max_len. */
int dc_conv_silu_l2(dc_ctx* ctx, void* stream, const float* p, const float* prev, const float* w, float* q, float* k,
                    float* v, uint32_t t, uint32_t ldp, uint32_t nk, uint32_t nv, uint32_t dk, uint32_t dv,
                    const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len);

/* ---- Conv::conv_state_update (kernels/conv.rs:38-46; spec cpu_ref.rs:86-95) ----
 * prev_out = the 3 raw rows that end this chunk of t rows, drawing on prev_in (NULL = zeros) when t < 3.
 * prev_out may be prev_in. */
int dc_conv_state_update(dc_ctx* ctx, void* stream, const float* p, const float* prev_in, float* prev_out,
                         uint32_t t, uint32_t ldp, uint32_t conv_dim);

/* ---- Delta::gated_delta (kernels/delta.rs:53-100; spec cpu_ref.rs:101-129) ----
 * The gated delta rule over t rows, fp32: q,k [t,nk,dk], v and o [t,nv,dv]; a,b read from rows of stride
 * ldab (value head h at column h); a_log, dt_bias fp32 [nv]; state fp32 [nv][dv][dk]; state_in may be
 * state_out (NULL state_in = zero state); state_out is written only with write_state. dk = dv = 128.
 * Packed sequences: seq_start u32 [n_seq+1], states [n_seq][nv][dv][dk], max_len the longest sequence
 * (0 = unknown). The fast kernels are the chunk-64 form on tensor cores (scratch from the context's
 * workspace: reserve dc_gated_delta_scratch_bytes up front to keep a forward allocation-free); the
 * baseline is the reference's sequential recurrence. */
int dc_gated_delta(dc_ctx* ctx, void* stream, const float* q, const float* k, const float* v, const float* a,
                   const float* b, const float* a_log, const float* dt_bias, const float* state_in, float* state_out,
                   float* o, uint32_t t, uint32_t ldab, uint32_t write_state, uint32_t nk, uint32_t nv, uint32_t dk,
                   uint32_t dv, const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len);
size_t dc_gated_delta_scratch_bytes(uint32_t t, uint32_t n_seq, uint32_t nv);
/* Scratch dc_attention takes for packed batches (seq_start given): the transposed V of `rows` cache rows. */
size_t dc_attention_scratch_bytes(uint32_t rows, uint32_t n_seq, uint32_t nkv);

/* ---- Conv::conv_silu_l2 + Delta::gated_delta in one call (no single counterpart in the reference, which
 * encodes the two back to back: forward.rs:1214-1234) ----
 * Same arguments and results as dc_conv_silu_l2 followed by dc_gated_delta, but q, k, v never reach
 * memory: the chunked delta rule's first kernel applies the conv, SiLU and L2 norm to the raw rows of p
 * as it loads them. a and b are the gate columns of the same rows (row stride ldp). Available when
 * dc_conv_gated_delta_supported(ctx) (fast delta rule, tcgen05 engine, split 3); DC_UNSUPPORTED otherwise,
 * and the caller uses the two-call form. */
int dc_conv_gated_delta(dc_ctx* ctx, void* stream, const float* p, const float* prev, const float* w, const float* a,
                        const float* b, const float* a_log, const float* dt_bias, const float* state_in, float* state_out,
                        float* o, uint32_t t, uint32_t ldp, uint32_t write_state, uint32_t nk, uint32_t nv, uint32_t dk,
                        uint32_t dv, const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len);
int dc_conv_gated_delta_supported(dc_ctx* ctx);

/* ======================================================================================
 * Whole-model prefill: the host loop of Forward (crates/decide-engine/src/forward.rs:1129-1328)
 * in C++ over the entry points above, for a batch of packed requests.
 * ====================================================================================== */

/* Model dims: the reference compiles these in (crates/decide-engine/src/config.rs:4-37); here they
 * are given at creation. Layer l is full attention iff (l+1) % full_attn_interval == 0 (config.rs:39-41). */
typedef struct dc_dims {
    uint32_t hidden, n_layers;
    uint32_t nq, nkv, head_dim, rot_dim;          /* attention: q heads, kv heads, head dim, rotary dims */
    uint32_t gdn_nk, gdn_nv, gdn_dk, gdn_dv;      /* Gated DeltaNet: key heads, value heads, dims */
    uint32_t inter, vocab;
    uint32_t full_attn_interval;                  /* 4 */
    uint32_t attn_gate;                           /* 1: fused in-proj is q|gate|k|v with a sigmoid output gate; 0: q|k|v */
    uint32_t swiglu_block;                        /* gate|up interleave of w_gu, 16 (config.rs:31) */
    float eps;                                    /* 1e-6 */
    float rope_theta;
} dc_dims;

/* One layer's tensors in the reference's fused layouts (crates/decide-engine/src/convert.rs:204-245).
 * bf16 matrices are [out, in] row-major; small tensors are fp32. Unused members are NULL. */
typedef struct dc_layer_weights {
    const float* in_norm;    /* [hidden] zero-centred */
    const void* w_in;        /* linear layer: [conv_dim + value_dim + 2 nv, hidden] = qkv|z|b|a;
                                attention layer: [q|gate|k|v or q|k|v, hidden] */
    const void* w_out;       /* [hidden, value_dim] or [hidden, nq*head_dim] */
    const float* post_norm;  /* [hidden] zero-centred */
    const void* w_gu;        /* [2 inter, hidden], gate|up interleaved in blocks of swiglu_block rows */
    const void* w_down;      /* [hidden, inter] */
    const float* conv_w;     /* linear: [conv_dim, 4] */
    const float* a_log;      /* linear: [nv] */
    const float* dt_bias;    /* linear: [nv] */
    const float* gnorm;      /* linear: [dv] */
    const float* q_norm;     /* attention: [head_dim] zero-centred */
    const float* k_norm;     /* attention: [head_dim] zero-centred */
} dc_layer_weights;

typedef struct dc_model dc_model;

/* Borrows the weights (device pointers, which must outlive the model), allocates every activation
 * buffer for up to max_rows packed rows, max_seqs requests and max_answers answer rows of up to
 * max_cand candidates each (Forward::new, forward.rs:1336-1379). NULL on failure (see dc_last_error). */
dc_model* dc_model_create(dc_ctx* ctx, const dc_dims* dims, const dc_layer_weights* layers, const void* embed,
                          const float* final_norm, uint32_t max_rows, uint32_t max_seqs, uint32_t max_answers,
                          uint32_t max_cand);
void dc_model_destroy(dc_model* m);
size_t dc_model_activation_bytes(dc_model* m);

/* One batched prefill from HOST buffers (the analogue of Forward::logits, forward.rs:704-731):
 * ids u32 [rows] packed by request, seq_start u32 [n_seq+1] (seq_start[0] = 0), ans_rows u32 [n_ans]
 * packed row index of each answer row, cand u32 [n_ans,max_cand], ncand u32 [n_ans]. Copies in, runs
 * all layers and the candidate-row head on `stream`, copies fp32 logits [n_ans,max_cand] out and waits.
 * Non-finite logits are an error (forward.rs:906-913). */
int dc_model_prefill(dc_model* m, void* stream, const uint32_t* ids, const uint32_t* seq_start, uint32_t n_seq,
                     const uint32_t* ans_rows, const uint32_t* cand, const uint32_t* ncand, uint32_t n_ans,
                     float* logits);

/* The same pass over the inputs left on the device by the last dc_model_prefill of this batch:
 * only enqueues (no copies, no wait); the logits stay in the model's device buffer. seq_start, n_seq
 * and n_ans must be that batch's (DC_INVALID_ARG otherwise). */
int dc_model_forward_resident(dc_model* m, void* stream, const uint32_t* seq_start, uint32_t n_seq, uint32_t n_ans);

/* CUDA graphs (on by default; DECIDE_GRAPHS=0 at creation or on = 0 turn them off): a batched forward of a
 * shape (rows, requests, longest request, answer rows, switches) that has run before is replayed from a graph
 * captured on its first run, on a stream the model owns that is joined to the caller's by events; the
 * first run of a shape is enqueued kernel by kernel and also captures. A single request is a few hundred
 * short kernels, which the host cannot enqueue as fast as the GPU runs them. Per-op profiling, a layer
 * limit, tensor-parallel shards and the chunked / snapshot route always run eagerly. Results are the same
 * bits either way. dc_model_graph_count: graphs held (at most 64; further shapes run eagerly). */
int dc_model_set_graphs(dc_model* m, uint32_t on);
size_t dc_model_graph_count(dc_model* m);

/* Work skipping, both on by default as in the reference:
 *  - truncation (forward.rs:830-831): a request is run only up to its last answer row; rows after it
 *    cannot reach a logit. A request without answer rows runs whole.
 *  - last-layer pruning (Forward::set_pruning, forward.rs:517-522, 1150-1186): when the last layer is
 *    full attention, only its K/V are computed for every row; the q|gate projection, attention,
 *    output projection, MLP and head run for the answer rows alone.
 * Results must not depend on either switch beyond fp32 rounding. */
int dc_model_set_pruning(dc_model* m, uint32_t on);
int dc_model_set_truncation(dc_model* m, uint32_t on);
/* Rows the last dc_model_prefill ran after truncation. */
uint32_t dc_model_resident_rows(dc_model* m);

/* Chunked prefill of ONE request (Forward::set_chunk, forward.rs:504-510, 919-942): with rows > 0 a
 * batch of a single request runs in chunks of at most `rows` rows, chunk-major (all layers of a chunk,
 * then the next chunk); Gated DeltaNet layers carry their 3 raw conv rows and their recurrent state
 * from chunk to chunk, attention layers append each chunk's K/V rows to a cache of their own and attend
 * over rows 0..=position. Results must not depend on the chunk size beyond fp32 rounding. rows = 0
 * (default) runs requests whole. Batches of several requests always run whole. Allocates the carried
 * state on first use (call it at set-up, not inside a request). Not available on a tensor-parallel shard. */
int dc_model_set_chunk(dc_model* m, uint32_t rows);
/* The prefix snapshot (Forward::build_snapshot, forward.rs:645-673, 237-247): runs the n prefix token ids
 * (host memory) once and keeps every layer's state after them (per linear layer conv rows + recurrent
 * state, per attention layer its K/V rows). A later single-request dc_model_prefill whose ids begin with
 * that prefix, that is longer than it and whose answer rows all lie past it restores the state and runs
 * only the remaining rows; any other request runs in full. n = 0 drops the snapshot. Synchronises. */
int dc_model_build_snapshot(dc_model* m, void* stream, const uint32_t* prefix_ids, uint32_t n);
/* Route of the last dc_model_prefill (Route, forward.rs:196-206): 0 = every row was run, 1 = it started
 * from the prefix snapshot, 2 = it started from a cached state. dc_model_last_start: the first row it
 * computed (Forward::last_start, forward.rs:686-692). */
uint32_t dc_model_last_route(dc_model* m);
uint32_t dc_model_last_start(dc_model* m);

/* The state cache for follow-up questions (forward.rs:704-731, 845-905). On the snapshot route, a
 * request whose ids hold the state marker between the prefix and its first answer row leaves the state
 * after the marker (every layer's conv rows, recurrent state and K/V rows up to there) in the cache,
 * evicting the least recently used entry when `entries` are held. A later request that starts with
 * exactly the ids an entry was captured from, and whose answer rows lie at or past their end, restores
 * that state and runs only the rows after it (route 2); among several such entries the longest wins.
 * Capacity 2 and the marker {550, 39087, 10485, 198} at creation (DEFAULT_STATE_ENTRIES, STATE_MARKER,
 * forward.rs:70-75). An entry's memory (each linear layer's state + K/V rows of the state's length) is
 * allocated when a state is first captured into it: that request allocates, later ones reuse it.
 * Results must not depend on the cache beyond fp32 rounding. */
#define DC_MAX_STATE_ENTRIES 4u
int dc_model_set_state_cache(dc_model* m, uint32_t entries);               /* Forward::set_state_cache, forward.rs:735; 0 = off */
void dc_model_forget_states(dc_model* m);                                   /* Forward::forget_states, forward.rs:749 */
uint32_t dc_model_state_cache_capacity(dc_model* m);                        /* forward.rs:755 */
uint32_t dc_model_cached_states(dc_model* m, uint32_t* lens, uint32_t cap); /* Forward::cached_states, forward.rs:761; returns the count */
int dc_model_set_state_marker(dc_model* m, const uint32_t* ids, uint32_t n); /* Forward::set_state_marker, forward.rs:767; empties the cache */

/* Runs only the first `n` layers and skips the head when n < n_layers (0 restores all layers): the
 * residual stream after layer n-1 is then in buffer "x" (debug_layers, forward.rs:778-797). While a
 * limit is set, pruning and truncation are off: every row of the residual is computed. */
int dc_model_set_layer_limit(dc_model* m, uint32_t n);
/* Device address of a named activation buffer: "x" (fp32 residual [rows,hidden]), "h", "p", "g",
 * "mlp", "xs", "logits". */
void* dc_model_buffer(dc_model* m, const char* name);
/* Waits for the device, then copies the first `bytes` bytes of that buffer to host memory `dst`. */
int dc_model_read_buffer(dc_model* m, const char* name, void* dst, size_t bytes);

/* Per-op timing table (the reference's DECIDE_PROFILE_PERKERNEL, crates/decide-metal/src/profile.rs:29-101):
 * when on, every op of a forward is bracketed by CUDA events; dc_model_profile synchronises, writes
 * "name total_ms calls" lines (largest first) into buf, clears the table and returns the text length. */
int dc_model_set_profiling(dc_model* m, uint32_t on);
size_t dc_model_profile(dc_model* m, char* buf, size_t len);

#ifdef __cplusplus
}
#endif
#endif /* DECIDE_CUDA_H */
