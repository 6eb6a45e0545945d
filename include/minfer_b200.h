/*
 * minfer_b200.h - C ABI of the B200-native (sm_100a) quantized decode path.
 *
 * This is the boundary a host program binds to (C, C++, ctypes, cgo ...): plain
 * pointers and sizes, no C++ or framework types.  The reference engine
 * (123-code/nano-inference, "minfer") has no plugin API; its seam between host
 * driver and CUDA kernels is the set of kernel launches in src/cuda_infer.cu
 * and the device functions of src/mega.cu.  Each entry point below names the
 * reference code it stands in for (paths relative to the reference root).
 *
 * Conventions
 *  - Every function returns an int status (MI_OK == 0).  Nothing here calls
 *    exit() or traps; mi_last_error() gives a text for the last failure on a
 *    context.  The reference's CK()/REQUIRE() print-and-exit behaviour
 *    (src/cuda_infer.cu:20, src/mega.cu:46-47) stays in the driver programs.
 *  - Pointers named *_dev are device pointers on the context's GPU; pointers
 *    named *_host are ordinary host memory.  Work is enqueued on the context's
 *    stream and is asynchronous unless stated otherwise.
 *  - There is no CPU fallback: without a usable CUDA device every call fails.
 *  - Device-side waits (bulk-copy barriers, polls for another CTA's or GPU's
 *    data, peer flags) are bounded; when one gives up the kernel records MI_ERR_TIMEOUT in the
 *    context's device error word, which mi_ctx_sync() reports.
 */
#ifndef MINFER_B200_H
#define MINFER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MI_API __attribute__((visibility("default")))
#else
#define MI_API
#endif

enum {
    MI_OK = 0,
    MI_ERR_INVALID = 1,      /* bad argument (null pointer, shape not a multiple of 32, ...) */
    MI_ERR_CUDA = 2,         /* a CUDA runtime call failed; see mi_last_error */
    MI_ERR_NOMEM = 3,        /* device or host allocation failed */
    MI_ERR_TIMEOUT = 4,      /* a bounded device-side wait gave up */
    MI_ERR_IO = 5,           /* file could not be opened / read */
    MI_ERR_FORMAT = 6,       /* GGUF file malformed or missing a tensor / key */
    MI_ERR_UNSUPPORTED = 7,  /* tensor type or shape outside what this path implements */
    MI_ERR_LIMIT = 8         /* request exceeds a fixed capacity stated by the entry point */
};

typedef struct mi_ctx mi_ctx;        /* one GPU: stream, error word, scratch */
typedef struct mi_weight mi_weight;  /* q4_0 matrix (or stack of equal matrices) in the tiled device layout */

/* ---- context ------------------------------------------------------------- */

/* Library version string. */
MI_API const char* mi_version(void);
/* Text for a status code. */
MI_API const char* mi_strerror(int status);

/* Create a context on CUDA device `device` with its own non-blocking stream.
 * Stands in for the reference's implicit process-wide state (one device, one
 * stream: src/cuda_infer.cu:1089, src/mega.cu:1149). */
MI_API int mi_ctx_create(int device, mi_ctx** out);
MI_API int mi_ctx_destroy(mi_ctx* ctx);
/* Use a caller-owned cudaStream_t (passed as void*) for all later work; NULL
 * restores the context's own stream.  The legacy default stream, whose handle is
 * 0, is selected with its alias cudaStreamLegacy ((void*)1). */
MI_API int mi_ctx_set_stream(mi_ctx* ctx, void* cuda_stream);
/* Wait for the stream, then report the device error word (MI_ERR_TIMEOUT if a
 * bounded wait gave up) and clear it. */
MI_API int mi_ctx_sync(mi_ctx* ctx);
MI_API const char* mi_last_error(const mi_ctx* ctx);
/* Time budget, in nanoseconds of the GPU's global timer, of every device-side wait of the
 * decode kernel (a consumer polling for another CTA's or another GPU's tagged words); default
 * 2 s.  When a wait runs out the kernel stops, drains its outstanding bulk copies and records
 * MI_ERR_TIMEOUT; mi_ctx_sync reports it and the next call starts clean.  The reference spins
 * without a bound (src/mega.cu:126-134); a bounded wait with a status has no counterpart there. */
MI_API int mi_ctx_set_wait_budget_ns(mi_ctx* ctx, unsigned long long ns);
/* Number of SMs the context sizes its grids for. */
MI_API int mi_ctx_sm_count(const mi_ctx* ctx);

/* Plain device memory for callers that have no CUDA binding of their own
 * (activations, logits).  mi_memcpy_* are synchronous on the context's stream. */
MI_API int mi_device_malloc(mi_ctx* ctx, size_t bytes, void** out_dev);
MI_API int mi_device_free(mi_ctx* ctx, void* ptr_dev);
MI_API int mi_memcpy_to_device(mi_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
MI_API int mi_memcpy_to_host(mi_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);

/* ---- machine probes ------------------------------------------------------ */

/* Read-only streaming bandwidth of this GPU as the kernels here stream: the call allocates `bytes`
 * of device memory (use several GB: far more than the L2), reads it `repeats` times in one launch
 * each and returns the best GB/s.  variant 0: 16-byte loads, eight in flight per thread; variant 1:
 * the GEMV's transport (per-warp ring of 4608-byte bulk copies).  The method of the reference's
 * bench/roofline.cu:39-116. */
MI_API int mi_probe_read_bw(mi_ctx* ctx, size_t bytes, int variant, int repeats, float* gbs_out);
/* One-way latency, in nanoseconds at the nominal SM clock, of an 8-byte word stored by one SM until
 * a polling SM sees it (two CTAs answering each other `iters` times): the cost of a phase boundary
 * of the decode kernel.  Stands where the reference measures its grid barrier
 * (bench/roofline.cu:125-149). */
MI_API int mi_probe_hop_ns(mi_ctx* ctx, int iters, float* ns_out);

/* ---- detokenizer (host only) ------------------------------------------------ */
/* Decode one vocabulary piece of a byte-level BPE tokenizer (the strings of tokenizer.ggml.tokens in a Qwen2 file) into
 * the text bytes it stands for: every code point of the piece maps back to one byte through the inverse of GPT-2's
 * byte-to-unicode table.  Replaces build_byte_decoder / detok_piece (src/detok.h:13-41).  Writes at most cap bytes to out
 * and returns the number of bytes of the decoded piece (never more than n); -1 on a null argument.  Needs no GPU. */
MI_API int64_t mi_detok_piece(const char* piece, int64_t n, char* out, int64_t cap);

/* ---- weights: GGUF q4_0 -> tiled device layout --------------------------- */

/* Upload `count` consecutive row-major q4_0 matrices of rows x cols (18-byte
 * blocks exactly as stored in a GGUF file: src/gguf.h:29,94-102) from host
 * memory and repack them ON THE DEVICE into the tiled layout the kernels
 * stream (32-row groups x kb-block tiles, nibbles then fp16 scales, each tile
 * one contiguous 16-byte-multiple run so a single bulk copy fetches it).
 * Replaces the host-side repack loops dt_q4r (src/cuda_infer.cu:761-777) and
 * pack_q4 (src/mega.cu:966-984).  cols must be a multiple of 32. Synchronous. */
MI_API int mi_weight_upload_q4_0(mi_ctx* ctx, const void* raw_host, int64_t rows, int64_t cols,
                                 int64_t count, mi_weight** out);
/* Same, the raw blocks already being in device memory (2-byte aligned). */
MI_API int mi_weight_repack_q4_0_dev(mi_ctx* ctx, const void* raw_dev, int64_t rows, int64_t cols,
                                     int64_t count, mi_weight** out);
/* Inverse of the repack: tiled layout back to GGUF block order in host memory
 * (count*rows*(cols/32)*18 bytes).  For round-trip checks. Synchronous. */
MI_API int mi_weight_download_q4_0(mi_ctx* ctx, const mi_weight* w, void* raw_host);
MI_API int mi_weight_free(mi_ctx* ctx, mi_weight* w);
/* Re-quantize a matrix stored as ggml Q4_1 (type 3), Q8_0 (8) or Q6_K (14) blocks into row-major q4_0 blocks, both in
 * device memory: src is rows x cols in its stored block format (rows contiguous), dst receives rows*(cols/32)*18 bytes
 * that mi_weight_repack_q4_0_dev accepts.  Dequantization per src/gguf.h:103-140, then the reference loader's symmetric
 * rule d = amax/7, q = clamp(lrintf(y/d) + 8, 0, 15), fp16 d (src/mega.cu:924-936; the same as src/cuda_infer.cu:814-842).
 * Replaces the host loop q4_rows (src/mega.cu:986-993), bit for bit.  cols must be a multiple of the block (32; 256 for
 * Q6_K).  Asynchronous on the context's stream. */
MI_API int mi_requant_q4_0(mi_ctx* ctx, int ggml_type, const void* src_dev, int64_t rows, int64_t cols, void* dst_dev);
/* Shape queries: rows, cols, count, bytes held on the device. */
MI_API int mi_weight_info(const mi_weight* w, int64_t* rows, int64_t* cols, int64_t* count, int64_t* device_bytes);

/* ---- activation quantizer ------------------------------------------------ */

/* q8_0 quantizer for M vectors of n floats (n a multiple of 32), each block of
 * 32: a = max|x|, xq = rint(x * 127/a) as int8, xd = fp16(a/127); a == 0 gives
 * zeros.  x_dev is [M][n], xq_dev [M][n], xd_dev [M][n/32] (fp16 bits).
 * Replaces quant_x_q8 / quant_x_q8_batch (src/cuda_infer.cu:80-89, 168-178). */
MI_API int mi_quant_q8(mi_ctx* ctx, const float* x_dev, int64_t n, int M, int8_t* xq_dev, uint16_t* xd_dev);

/* ---- q4_0 x q8_0 GEMV ---------------------------------------------------- */

/* y[c][r] = sum_b dw[c][r][b] * dx[b] * (sum_k n_k*xq_k - 8*sum_k xq_k) + bias[r]
 * for every matrix c of the stack; the integer part is exact, every block product
 * dw*dx*isum is exact in double, the sum is carried in double and rounded to fp32
 * once, so the result does not depend on how the blocks are split or ordered.  xq_dev [cols], xd_dev [cols/32] fp16 bits, bias_dev [rows] or
 * NULL, y_dev [count][rows] fp32.  One launch covers the whole stack.
 * Replaces gemv_dp4a (src/cuda_infer.cu:94-127) and row_dot (src/mega.cu:178-196). */
MI_API int mi_gemv_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                         const float* bias_dev, float* y_dev);
/* Same with explicit tuning: ksplit (0 = automatic) is the number of K-splits
 * per 32-row group, variant (0 = default) selects a warps/stages instantiation. */
MI_API int mi_gemv_q4_q8_ex(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                            const float* bias_dev, float* y_dev, int ksplit, int variant);
/* The exact integer block sums isum[r][b] = sum n*xq - 8*sum xq (int32,
 * [rows][cols/32]) of matrix 0 of the stack, produced by the same unpack + dp4a
 * code as the GEMV.  For bit-exact parity checks. */
MI_API int mi_block_isums_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, int32_t* isum_dev);

/* Same product as mi_gemv_q4_q8, for callers that must not allocate device memory
 * once they are running: a serving loop whose whole memory budget was handed to
 * another allocator at start-up (a later cudaMalloc could fail, or stall every
 * stream of the device while it runs), or a host that audits its plugins and
 * forbids allocation after initialisation.  mi_gemv_q4_q8 grows a scratch buffer
 * with cudaMalloc the first time a shape needs K-splitting; this entry point never
 * does.  Its split-K scratch (partial sums and arrival counters) is a fixed array
 * inside the library image: 65536 partial sums and 2048 counters, 528 KB that every
 * GPU which loads the library holds until the process exits.  A call whose stack
 * needs more (row groups x K-splits x 32 > 65536, or more than 2048 row groups
 * over the whole stack when it is K-split) returns MI_ERR_LIMIT and does nothing
 * (the shared scratch is not touched either).
 * It calls no cudaMalloc, cudaFree or other allocating routine.
 * The first call on a device looks the array's device address up (one symbol
 * query, made with the context's device current; the calling thread's current
 * device is put back before the call returns); make that first call before any
 * stream capture begins.  First calls from several host threads are serialized
 * by the library.  All calls share the one array and it keeps whatever the last
 * call left in it (the counters are cleared at the start of every call): two calls
 * that overlap on the GPU - different streams, or different contexts on the same
 * device - race on it and give wrong results; serialize them.
 * This entry point has no counterpart in the reference. */
MI_API int mi_gemv_q4_q8_noalloc(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                                 const float* bias_dev, float* y_dev);

/* ---- q4_0 x q8_0 GEMM for multi-token steps ---------------------------------- */

/* Y[m][r] = the GEMV sum of row r against token vector m, for M = 1..16 token vectors in
 * one pass over the weights (speculative verify, chunked prefill, small batches).  The
 * integer block dot products run on the tensor cores (tcgen05.mma.kind::i8, one K=32 MMA
 * per q4_0 block, int32 accumulators in tensor memory), the per-block fp16 scaling on the
 * CUDA cores with the GEMV's own expression, so Y[m] carries exactly the bits
 * mi_gemv_q4_q8 gives for xq[m] alone, whatever M is.  xq_dev [M][cols] int8, xd_dev
 * [M][cols/32] fp16 bits, y_dev [M][rows] fp32; w must be a single matrix (count == 1).
 * Replaces gemv_dp4a_batch<T> (src/cuda_infer.cu:183-222, T <= 8) and the mma.sync path
 * tile_dot (src/mega.cu:197-244). */
MI_API int mi_gemm_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev, int M,
                         const float* bias_dev, float* y_dev);

/* Host-buffer convenience: quantize x_host [cols] on the device, run the GEMV on
 * matrix stack w, and copy y back to y_host [count][rows].  Host-to-device and
 * device-to-host copies are inside the call; it returns when y_host is valid. */
MI_API int mi_gemv_q4_f32_host(mi_ctx* ctx, const mi_weight* w, const float* x_host, const float* bias_dev,
                               float* y_host);

/* ---- model and decode loop -------------------------------------------------- */

typedef struct mi_model mi_model;    /* weights (tiled), fp16 KV cache and decode state of one Qwen2-architecture model */

typedef struct mi_model_config {
    int32_t n_layer, n_embd, n_ff, n_head, n_head_kv, head_dim, n_vocab, max_seq, tied_lm_head, grid_ctas;
    float rope_base, rms_eps;
    int64_t q4_weight_bytes_per_token;   /* q4_0 bytes every decoded token streams (18 bytes per 32 weights) */
    int64_t kv_bytes_per_position;       /* fp16 K+V bytes per cached position over all layers */
} mi_model_config;

enum { MI_DECODE_PERSISTENT = 0,   /* one cooperative launch: all phases, layers and steps in one persistent kernel */
       MI_DECODE_PER_PHASE = 1 };  /* the same kernel launched once per phase (stream order between the phases) */

/* MI_STATE_H: residual stream at the input of the layer whose QKV phase ran last;
 * MI_STATE_H_MID: residual stream after the attention block of the layer whose gate/up phase ran last. */
enum { MI_STATE_H = 0, MI_STATE_Q = 1, MI_STATE_ATT = 2, MI_STATE_KCACHE = 3, MI_STATE_VCACHE = 4,
       MI_STATE_ACT_Q = 5, MI_STATE_ACT_D = 6,
       MI_STATE_PROFILE = 7,
       MI_STATE_H_MID = 8 };  /* 32 x uint64 nanoseconds per phase part on CTA 0, filled when the model was loaded
                                 * with MINFER_PROFILE set in the environment: slots 2k / 2k+1 = staging / work of phase
                                 * kind k (0 QKV, 1 attention, 2 O, 3 gate-up, 4 down, 5 lm_head), 12 = waiting for other CTAs' data,
                                 * 13 = per-step prologue, 18..22 = tile loops (loop, ring wait, arithmetic, issuing copies; 19 =
                                 * fold + epilogue), 23..28 = parts of the norm prologue; on an attention CTA (MINFER_PROFILE_CTA)
                                 * 14..17 and 27..31 = parts of the attention; slots 8 and 9 of the persistent engine hold the
                                 * launch's SM cycles and nanoseconds.  The reference's PROFILE=1 (src/mega.cu:111-119). */

/* Load a Qwen2-architecture GGUF file (metadata keys and tensor names
 * exactly as the reference drivers read them: src/cpu_infer.cpp:71-98), repack
 * every matrix on the device (q/k/v fused, rows of q and k made pair-adjacent for
 * RoPE; gate and up interleaved by 32-row group), allocate an fp16 KV cache for
 * max_seq positions and plan the per-phase work split.  output.weight may be
 * absent or byte-identical to token_embd.weight (tied lm_head, stored once).
 * Replaces the load / upload / buffer set-up of src/cuda_infer.cu:846-955 and
 * src/mega.cu:1067-1139.  Matrices stored as Q4_1, Q8_0 or Q6_K are re-quantized
 * to q4_0 on the device first (mi_requant_q4_0), as the reference's loader does on
 * the host (src/mega.cu:986-993, 1109); a Q8_0 token embedding is kept and read as
 * stored (src/mega.cu:639-646, 1110-1111).  Other matrix types, and norms or biases
 * that are not F32, give MI_ERR_UNSUPPORTED. */
MI_API int mi_model_load_gguf(mi_ctx* ctx, const char* path, int max_seq, mi_model** out);
MI_API int mi_model_free(mi_ctx* ctx, mi_model* model);
MI_API int mi_model_info(const mi_model* model, mi_model_config* out);
/* Device address (and size) of one state buffer, for inspection by tests. */
MI_API int mi_model_state_ptr(const mi_model* model, int which, void** ptr, int64_t* bytes);

/* Run n_steps decode steps at positions pos0 .. pos0+n_steps-1.  Step s takes
 * in_tokens_host[s] while s < n_forced (prompt / teacher forcing), afterwards the
 * previous step's greedy token; out_tokens_host[s] receives the greedy token after
 * step s (lowest index on ties, as src/cpu_infer.cpp:153-154).  logits_dev, if not
 * NULL, receives [n_steps][n_vocab] fp32 logits.  elapsed_ms, if not NULL, receives
 * the device time of the steps (CUDA events on the context's stream).  Returns
 * after the steps have finished.  Replaces the record() step graph + decode loop of
 * src/cuda_infer.cu:1031-1201 and the mega kernel of src/mega.cu:597-903. */
MI_API int mi_decode(mi_ctx* ctx, mi_model* model, const int32_t* in_tokens_host, int n_forced, int n_steps, int pos0,
                     int32_t* out_tokens_host, float* logits_dev, int mode, float* elapsed_ms);

/* Stop rule of text generation.  Once set (token >= 0), a run of whole steps ends after the first step whose prediction
 * is consumed as the next input (not a forced position) and equals `token`: the persistent kernel leaves its loop on
 * every CTA (src/mega.cu:868-874, done = stop_eos && cur == eos), the kernel-sequence engine looks at each token before
 * it launches the next step (src/cuda_infer.cu:1186-1193), mi_generate_spec stops emitting (src/cuda_infer.cu:1254-1275).
 * The stop token itself is the last token produced.  mi_model_last_count: how many tokens the last mi_decode or
 * mi_generate_spec call produced (a run through mi_decode_run reports through its ring's count).  -1 switches the rule
 * off (the default: the id-printing form of the drivers never stops early, src/mega.cu:1017). */
MI_API int mi_model_set_stop_token(mi_model* model, int token);
MI_API int mi_model_last_count(const mi_model* model);
/* Top-1 minus top-2 logit of each of the first n steps of the last mi_decode call on this model
 * (host memory out).  The reference's engine reports this margin per token (src/mega.cu:385-392,
 * 523-550, printed at :1189, 1196, 1241); its A/B harness reads it (tools/ab.sh:41,49). */
MI_API int mi_decode_margins(mi_ctx* ctx, mi_model* model, int n, float* margins_host);

/* ---- streaming hand-off of generated tokens ----------------------------------- */

/* A token ring: pinned host memory mapped into the GPU's address space.  A generation started with
 * mi_decode_run publishes every step's greedy token, its logit margin and a GPU time stamp into the
 * ring while the kernel is still running (the count of valid entries is raised every fourth step
 * and at the end, after a system-scope fence); the host polls mi_ring_peek and can print or stop
 * reading at any time.  The reference's mega driver does exactly this: src/mega.cu:1130-1137 (the
 * mapped ring), :847-856 (publish), :1166-1178 (host poll).  Entries accumulate over successive
 * runs until mi_ring_reset; a run that would overflow the ring is refused with MI_ERR_LIMIT. */
typedef struct mi_token_ring mi_token_ring;
MI_API int mi_ring_create(mi_ctx* ctx, int capacity, mi_token_ring** out);
MI_API int mi_ring_destroy(mi_ctx* ctx, mi_token_ring* ring);
/* Waits for the stream, then forgets all entries. */
MI_API int mi_ring_reset(mi_ctx* ctx, mi_token_ring* ring);
/* Number of valid entries right now (acquire load) and the arrays they live in (host pointers,
 * valid for the ring's lifetime): tokens, margins, GPU nanosecond stamps.  Any pointer may be NULL. */
MI_API int mi_ring_peek(const mi_token_ring* ring, int* count, const int32_t** tokens, const float** margins,
                        const uint64_t** ns);
/* mi_decode with the persistent engine, asynchronous: enqueue n_steps steps at positions pos0..,
 * return at once; the tokens arrive in `ring`.  mi_ctx_sync waits for the end (and reports a
 * time-out).  The proposal of the reference-side boundary, mi_decode_run(ctx, model, prompt,
 * n_prompt, n_gen, ring), in this library's argument convention. */
MI_API int mi_decode_run(mi_ctx* ctx, mi_model* model, const int32_t* in_tokens_host, int n_forced, int n_steps, int pos0,
                         mi_token_ring* ring);

/* Test hook for the time-out path: from now on the producers of phase `phase` (5 * layer + kind;
 * 5 * n_layer = lm_head) compute but publish nothing, so the waits of that phase's consumers run
 * out after the context's wait budget and the call returns MI_ERR_TIMEOUT - nothing hangs or
 * faults.  -1 restores normal operation.  No counterpart in the reference. */
MI_API int mi_model_debug_drop_phase(mi_model* model, int phase);
/* Run phases [phase_begin, phase_end) of one step (5 per layer: QKV, attention, O,
 * gate/up, down; then the lm_head) one launch each, leaving the state buffers for
 * inspection.  For per-phase parity checks. */
MI_API int mi_decode_phases(mi_ctx* ctx, mi_model* model, int32_t token, int pos, int phase_begin, int phase_end);

/* ---- the M-token step ----------------------------------------------------------- */

/* Scores M (1..16) tokens at positions pos0 .. pos0+M-1 in ONE pass over the weights:
 * token i is processed as if it were decoded alone after tokens 0..i-1 of the call, so
 * its logits do not depend on M (the drafted-token verify step of the reference,
 * src/cuda_infer.cu:990-1029 forward_batch and src/mega.cu:246-299 gemv_seq; also its chunked
 * prompt processing, src/cuda_infer.cu:1130-1144).  Projections run as mi_gemm_q4_q8, attention
 * as mi_attn_splitkv over the model's fp16 KV cache, which receives all M positions; a caller
 * that accepts only a prefix simply continues at the first rejected position.
 * out_tokens_host[i] (optional) = greedy token after token i; logits_dev (optional) = [M][n_vocab]
 * fp32.  The model's current token becomes out_tokens[M-1].  Synchronous.  Unsharded models only. */
MI_API int mi_verify(mi_ctx* ctx, mi_model* model, const int32_t* tokens_host, int M, int pos0,
                     int32_t* out_tokens_host, float* logits_dev, float* elapsed_ms);

/* Greedy generation with lossless n-gram speculation: process the prompt (16 tokens per weight
 * pass), then generate n_gen tokens.  Each step drafts up to draftk (0..15; 0 = no speculation)
 * tokens by prompt lookup - the tokens that followed the latest earlier occurrence of the last
 * ngmax .. 1 tokens of the sequence so far - scores the current token and the draft in ONE
 * M-token pass (mi_verify) and keeps the longest prefix of the draft that equals the model's own
 * greedy tokens; without a draft it runs one single-token step (mi_decode).  How many of the drafted
 * tokens a step submits is decided per step, as in the reference's kernel (src/mega.cu:579-589): the
 * length that maximizes expected tokens per unit of time for the running acceptance estimate, priced
 * with the device times the loop has measured for its own two kinds of step - none, where a pass of
 * that size costs more than it is expected to bring (every 32nd such step still tests one token).
 * draftk < 0: always submit the whole draft (up to -draftk tokens), whatever it costs.  Because a token's
 * logits are the same bits in both kinds of step, out_tokens_host[0 .. n_gen) is exactly the
 * sequence plain greedy decoding produces (the first id is the prediction after the last prompt
 * token).  margins_host (optional, [n_gen]): the logit margin (top-1 minus top-2) of the step that
 * produced each id.  stats (optional, 4 values): generation steps, drafted tokens, accepted tokens,
 * steps that ran a draft.  The reference's speculative loops: src/cuda_infer.cu:1203-1292 (host) and
 * src/mega.cu:557-589, 863-895 (in-kernel); its gate tools/specbench.sh:33-36. */
MI_API int mi_generate_spec(mi_ctx* ctx, mi_model* model, const int32_t* prompt_host, int n_prompt, int n_gen, int ngmax,
                            int draftk, int32_t* out_tokens_host, float* margins_host, int64_t* stats);
/* Logit margins of the first n tokens of the last mi_verify pass on this model. */
MI_API int mi_verify_margins(mi_ctx* ctx, mi_model* model, int n, float* margins_host);

/* ---- batched decode of independent sequences ------------------------------------- */

/* A batch object owns n_slots KV-cache slabs of max_seq positions each (fp16, laid out like the
 * model's own cache) for sequences decoded together.  mi_batch_step runs ONE decode step for n
 * of them: sequence i has its current token tokens_host[i] at position positions_host[i] of slab
 * slots_host[i] (distinct slots within a call).  Up to 16 sequences share one pass over the
 * weights as columns of the M-token step (tcgen05 GEMM, one attention CTA set per column over
 * that column's own slab); more sequences run further passes.  Every column is processed exactly
 * as if it were alone: out_tokens_host[i] and logits_dev[i][n_vocab] are the bits a batch-1 decode
 * of that sequence gives.  Prompts enter the same way, one token per step and sequence (or through
 * mi_verify on the model's own cache for a single sequence).  The reference has no independent-
 * sequence batching (README.md:54); its closest code is gemv_dp4a_batch<T>
 * (src/cuda_infer.cu:183-222). */
typedef struct mi_batch mi_batch;
MI_API int mi_batch_create(mi_ctx* ctx, mi_model* model, int n_slots, int max_seq, mi_batch** out);
MI_API int mi_batch_free(mi_ctx* ctx, mi_batch* batch);
MI_API int mi_batch_step(mi_ctx* ctx, mi_batch* batch, int n, const int32_t* tokens_host, const int32_t* slots_host,
                         const int32_t* positions_host, int32_t* out_tokens_host, float* logits_dev, float* elapsed_ms);

/* Split-KV causal attention with grouped queries for M (1..16) consecutive query positions
 * (replaces attn_partial + attn_combine, src/cuda_infer.cu:650-702, and mega's attention + combine,
 * src/mega.cu:414-521, 705-741).  q_dev: [M][n_head * head_dim] fp32 in natural dimension order
 * (after RoPE); kcache_dev / vcache_dev: fp16 bits, [positions][n_head_kv * head_dim], holding
 * positions 0 .. pos0+M-1; query i attends to positions 0 .. pos0+i.  Scores are scaled by
 * 1/sqrt(head_dim); the softmax merge across KV chunks uses the running-maximum rule of the
 * reference with sums carried in double.  out_dev: [M][n_head * head_dim] fp32.  Asynchronous
 * on the context's stream.  head_dim in {32, 64, 128}. */
MI_API int mi_attn_splitkv(mi_ctx* ctx, const float* q_dev, const uint16_t* kcache_dev, const uint16_t* vcache_dev,
                           int n_head, int n_head_kv, int head_dim, int pos0, int M, float* out_dev);

/* ---- tensor parallelism (one process per GPU) --------------------------------- */

/* The reference is single-GPU (README.md:54); this part has no counterpart in it.
 * The gate/up, down and lm_head jobs of the decode step (nine tenths of the weight bytes) are
 * sharded by rows: GPU `rank` of `world` owns a contiguous range of each matrix's 32-row groups
 * (mi_tp_partition) and streams only those rows.  What a sharded phase produces lands in a
 * buffer that all GPUs lay out identically, with the entries a GPU does not own left at zero;
 * an all-reduce (sum) of that buffer after the phase - NCCL, issued by the host program -
 * therefore reproduces, bit for bit, what one GPU computes (x + 0 is exact for every type).
 * The QKV and O projections and attention are computed in full by every GPU (no exchange).
 * Per token and layer: all-reduce after the gate/up phase (MI_TP_ACT) and after the down phase
 * (MI_TP_PART_DOWN); after the lm_head each GPU holds the best logit of its rows
 * (MI_TP_BEST: {float value, int32 token}); gather those and call mi_tp_pick.  MI_TP_QKV and
 * MI_TP_PART_O name buffers that need no exchange; they stay addressable for inspection. */
enum { MI_TP_QKV = 0, MI_TP_PART_O = 1, MI_TP_ACT = 2, MI_TP_PART_DOWN = 3, MI_TP_BEST = 4 };

/* Range [begin, end) of `groups` row groups owned by `rank`.  Pure arithmetic, no GPU needed. */
MI_API void mi_tp_partition(int groups, int rank, int world, int* begin, int* end);
/* mi_model_load_gguf for GPU `tp_rank` of `tp_world`. */
MI_API int mi_model_load_gguf_tp(mi_ctx* ctx, const char* path, int max_seq, int tp_rank, int tp_world, mi_model** out);
/* Device address and byte size of an exchanged buffer (layer is ignored where it does not apply). */
MI_API int mi_model_tp_region(const mi_model* model, int which, int layer, void** ptr, int64_t* bytes);
/* Enqueue phases [phase_begin, phase_end) of the step at position pos, one launch per phase, WITHOUT
 * waiting; the input token is the model's device-resident current token.  On a sharded model the
 * buffer a phase writes is zeroed first.  The caller interleaves its all-reduces on the same stream. */
MI_API int mi_decode_launch(mi_ctx* ctx, mi_model* model, int pos, int phase_begin, int phase_end);
/* The same range as ONE cooperative launch (the phases chained inside the kernel, as in the persistent loop): for a run of
 * phases with no exchange between them - on a sharded model QKV, attention, O and gate/up of a layer. */
MI_API int mi_decode_launch_fused(mi_ctx* ctx, mi_model* model, int pos, int phase_begin, int phase_end);
/* Exchange through peer memory instead of a collective library: every process calls mi_tp_ipc_handles (192 bytes out:
 * CUDA IPC handles of its activation buffer, partial-sum buffer and flag block), the host program gathers the handles of all
 * ranks ([world][192 bytes], rank order) and passes them to mi_tp_ipc_open.  From then on mi_tp_exchange(which, layer) - one
 * small kernel - stores this GPU's slice of MI_TP_ACT / MI_TP_PART_DOWN / MI_TP_BEST into every peer's buffer over NVLink,
 * flags the peers and waits (bounded; MI_ERR_TIMEOUT through mi_ctx_sync) for theirs; after MI_TP_BEST it also makes the
 * overall greedy token current.  Every GPU issues the same sequence of exchanges.  Same bits as the all-reduce path.
 * Once mi_tp_ipc_open has run, mi_decode(..., MI_DECODE_PERSISTENT, ...) works on the sharded model too - called with the
 * same arguments on every GPU, it runs the whole generation as one cooperative launch per GPU and does these exchanges
 * inside the kernel (every producing CTA stores its results into the peers' exchange blocks as well; consumers poll,
 * bounded). */
MI_API int mi_tp_ipc_handles(mi_ctx* ctx, mi_model* model, void* out_host);
MI_API int mi_tp_ipc_open(mi_ctx* ctx, mi_model* model, const void* all_host);
MI_API int mi_tp_exchange(mi_ctx* ctx, mi_model* model, int which, int layer);
/* Position argument of mi_decode_launch that means "the model's device-resident position": a launch sequence
 * enqueued with it does not depend on the step and can be captured once into a CUDA graph by the host program
 * (tensor-parallel steps: the phase launches and the NCCL all-reduces between them) and replayed per token. */
#define MI_POS_DEVICE (-1)
/* Set / add to (both asynchronously) the device-resident position. */
MI_API int mi_model_set_pos(mi_ctx* ctx, mi_model* model, int pos);
MI_API int mi_model_advance_pos(mi_ctx* ctx, mi_model* model, int delta);
/* Set (asynchronously) / read back (synchronously) the model's current token. */
MI_API int mi_model_set_token(mi_ctx* ctx, mi_model* model, int32_t token);
MI_API int mi_model_get_token(mi_ctx* ctx, mi_model* model, int32_t* token, float* best_val);
/* gathered_dev: [world] x {float, int32} as published under MI_TP_BEST by each GPU; makes the overall
 * greedy token (largest value, lowest id on ties) the current token. */
MI_API int mi_tp_pick(mi_ctx* ctx, mi_model* model, const void* gathered_dev, int world);

#ifdef __cplusplus
}
#endif
#endif /* MINFER_B200_H */
