/*
 * tiny_gemma_b200.h — C ABI of libtinygemma_b200.so
 *
 * B200 (sm_100a) implementation of tiny-gemma's int8 weight-only Gemma-3
 * inference path: prefill, decode and the greedy / min-p samplers. The
 * reference (fattorib/tiny-gemma) has no FFI of its own: its API is a set of
 * C++ free functions in headers. Each entry point below names the reference
 * function it stands in for (file:line within that project). The C++20 header
 * layer under tiny-gemma_b200/host/ re-creates the reference's own names
 * (gemma::forward_decode, ops::minp_logits, ...) on top of these calls.
 *
 * Conventions
 *   - every function returns 0 on success, a TG_E* code otherwise; nothing
 *     throws or aborts across this boundary; tg_last_error() returns the
 *     message of the calling thread's last failure;
 *   - pointers named *_host are ordinary host memory; no device pointers and
 *     no framework types cross the boundary except in the tg_dev_* calls,
 *     which take raw CUDA device pointers for callers that already hold data
 *     in HBM;
 *   - there is no CPU fallback: without a CUDA device every call fails with
 *     TG_ENODEVICE;
 *   - one tg_state is one batch of independent sequences on one GPU; a state
 *     is not thread-safe, different states are independent.
 */
#ifndef TINY_GEMMA_B200_H
#define TINY_GEMMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
	TG_OK = 0,
	TG_EINVAL = 1,    /* bad argument (null pointer, size out of range)             */
	TG_ENODEVICE = 2, /* no usable CUDA device                                      */
	TG_ECUDA = 3,     /* a CUDA runtime call failed; see tg_last_error()            */
	TG_EIO = 4,       /* weights file missing / short                               */
	TG_ESHAPE = 5,    /* K or N outside the supported set (static_switch.hpp:7-58)  */
	TG_ESTATE = 6,    /* call order violated (e.g. prefill on a non-empty cache)    */
	TG_ENOMEM = 7
};

/* config::Config, reference csrc/include/config.hpp:7-20 — same fields, same order */
typedef struct tg_config {
	int hidden_size;
	int intermediate_size;
	int n_layers;
	int n_vocab;
	int n_pos;
	int n_pos_local;
	int head_dim;
	int n_head;
	int n_kv;
	float rope_theta;
	float rope_theta_local;
	int window_pattern;
} tg_config;

typedef struct tg_model tg_model;
typedef struct tg_state tg_state;

const char *tg_last_error(void);
const char *tg_version(void);
int tg_device_count(int *count);

/* config::CONFIG_MAP.at(name), config.hpp:46-48: "270m" or "1B"; unknown name -> TG_EINVAL
 * (the reference throws std::out_of_range, gemma.cpp:38) */
int tg_config_by_name(const char *name, tg_config *out);

/* ---- model -------------------------------------------------------------- */

/* gemma::Transformer(Config), transformer.hpp:33-46. Allocates the weight
 * store in the HBM of `device`; weights are zero until loaded. */
int tg_model_create(const tg_config *cfg, int device, tg_model **out);
int tg_model_free(tg_model *m);

/* gemma::read_weights(Transformer*, const char*), transformer.hpp:99-165.
 * `gemma_i8.bin` layout exactly as py/gemma.py:27-77 writes it; the bytes are
 * placed in HBM unchanged. Missing file -> TG_EIO (reference: runtime_error);
 * a short file -> TG_EIO (the reference ignores short reads). */
int tg_model_load_file(tg_model *m, const char *path);
/* same, from a host buffer holding the file image */
int tg_model_load_memory(tg_model *m, const void *bytes_host, size_t nbytes);
/* expected size in bytes of gemma_i8.bin for this config */
int tg_model_file_bytes(const tg_config *cfg, size_t *nbytes);

/* decode::RoPE(Config*, is_sw), decode.hpp:118-134,176-201: the cos/sin tables
 * [n_pos, head_dim] are built by host code and handed over. is_local selects the
 * sliding-window (theta_local) table. n_pos must be at least the config's n_pos (the
 * reference always builds that many rows; the kernels read row `position`), else TG_EINVAL. */
int tg_model_set_rope(tg_model *m, int is_local, const float *cos_host, const float *sin_host, int n_pos);
/* lut::GeLUTable{min,max,size}, ops.hpp:22-51: table built on the host. */
int tg_model_set_gelu_table(tg_model *m, float min, float max, const float *table_host, int size);
/* builds both RoPE tables and a GeLU table of `gelu_size` entries over [-4,4]
 * with this library's own host code (same formulas as decode.hpp:176-201 and
 * ops.hpp:16-39) — what the C++ header layer does when the caller constructs
 * decode::RoPE / lut::GeLUTable itself. */
int tg_model_build_tables(tg_model *m, int gelu_size);

/* ---- decode state ------------------------------------------------------- */

/* decode::DecodeState(batch, Config*), decode.hpp:242-276: KV caches (512-slot
 * ring on local layers, max_pos_global slots on global layers; pass 0 for the
 * reference's n_pos) and activations for `batch` independent sequences. */
int tg_state_create(tg_model *m, int batch, int max_pos_global, tg_state **out);
int tg_state_free(tg_state *s);
/* empties every cache (position_ptr = buffer_ptr = 0) */
int tg_state_reset(tg_state *s);
/* KVCache::position_ptr of sequence b (decode.hpp:18) */
int tg_state_position(tg_state *s, int b, int *position);

/* gemma::forward_prefill, transformer.hpp:49-73. ids_host is [batch, n_tokens]
 * row-major; every sequence of the batch has the same prompt length. Needs
 * empty caches (decode.hpp:78-79) else TG_ESTATE. logits_host may be NULL;
 * otherwise receives [batch, n_vocab] fp32 for the last prompt position.
 * Batches of 4 and more are prefilled together (their rows stacked, up to 16384
 * rows per pass): a sequence's logits then agree with those of a
 * single-sequence state to rounding (the GEMMs tile and split other row counts
 * differently), not bit for bit; batches below 4 are prefilled one sequence
 * per pass and are bit-identical to it. */
int tg_prefill(tg_state *s, const int *ids_host, int n_tokens, float *logits_host);

/* gemma::forward_decode, transformer.hpp:75-97: one token per sequence.
 * ids_host NULL = feed the token the last tg_sample_* call produced (it is
 * still on the device). logits_host may be NULL. */
int tg_decode(tg_state *s, const int *ids_host, float *logits_host);

/* Continuation of a non-empty context (a further turn of a conversation): the n tokens of ids_host
 * are fed one after the other through the decode path, each seeing the cache the earlier ones left, so
 * the result equals n calls of forward_decode (transformer.hpp:75-97) on those tokens. The reference
 * cannot do this with its prefill — KVCache::update_prefill asserts an empty cache (decode.hpp:78-79,
 * listed as a limitation in README.md:96). One sequence per state; logits_host may be NULL, otherwise it
 * receives the logits after the last token. */
int tg_append(tg_state *s, const int *ids_host, int n, float *logits_host);

/* ops::argmax_logits, ops.hpp:744-760, on the logits of the last forward
 * (still in HBM): lowest index wins ties, NaN never wins, -1 if no logit is
 * above -inf. toks_host receives [batch] ids (may be NULL). */
int tg_sample_argmax(tg_state *s, int *toks_host);
/* ops::minp_logits, ops.hpp:762-859, on the logits of the last forward; one
 * uniform per sequence in randf_host[batch]. Like the reference it overwrites
 * the logits with its "probabilities". */
int tg_sample_minp(tg_state *s, float minp, float temp, const float *randf_host, int *toks_host);
/* copy the device logits buffer (after a forward or a sampler) to the host */
int tg_logits_read(tg_state *s, float *logits_host);

/* The decode loop of gemma::generate, transformer.hpp:226-250 (forward_decode
 * + sampler, n_steps times) run on the device without a host round trip per
 * token. first_ids_host[batch] is fed to the first step. minp >= 1 selects
 * argmax (transformer.hpp:229); else randf_host holds [n_steps, batch]
 * uniforms. toks_host receives [n_steps, batch]. Calls of up to 4096 tokens
 * (n_steps * batch) move ids, uniforms and tokens through the state's pinned
 * staging buffer and synchronise once, so n_steps = 1 per call is a per-token
 * loop with one launch and one synchronisation per token. An id outside the
 * vocabulary is TG_EINVAL. */
int tg_generate(tg_state *s, const int *first_ids_host, int n_steps, float minp, float temp, const float *randf_host,
                int *toks_host);

/* parity helpers: read back cache rows / the final-normed hidden state */
int tg_kv_read(tg_state *s, int b, int layer, int slot0, int nslots, float *k_host, float *v_host);
int tg_hidden_read(tg_state *s, float *hidden_host);

/* ---- isolated operators (host buffers) ---------------------------------- */

/* ops::linear_decode / ops::lm_head_decode, ops.hpp:634-667 -> gemv::launch_qgemv(_logits),
 * linalg.hpp:176-204: y[n] = scale[n] * sum_k x[k] * W[k,n]; W is [K,N] row-major int8.
 * K,N must be in the reference's supported set, else TG_ESHAPE. */
int tg_qmatvec(float *y_host, const float *x_host, const int8_t *w_host, const float *scales_host, int K, int N);
/* ops::linear_prefill, ops.hpp:618-632 -> gemm::launch_qgemm, linalg.hpp:298-308:
 * C[M,N] = scale[n] * (A[M,K] . W[K,N]) */
int tg_qgemm(float *c_host, const float *a_host, const int8_t *w_host, const float *scales_host, int M, int K, int N);
/* ops::argmax_logits / ops::minp_logits on a host logits buffer of n entries
 * (n = 262144 in the reference); minp mutates logits_host like the reference */
int tg_argmax_logits(const float *logits_host, int n, int *tok);
int tg_minp_logits(float *logits_host, int n, float minp, float temp, float randf, int *tok);
/* The last step of ops::minp_logits in isolation (ops.hpp:849-857, the inverse-CDF loop):
 * *idx = first i with fl(cum0 + p[0] + ... + p[i]) >= randf, the sum taken sequentially in fp32,
 * or -1 if it never gets there; *cum_out (may be null) = the running sum where the scan stopped.
 * The GPU evaluates the sequential chain exactly with a parallel scan; this entry exists so that
 * the exactness can be tested on arbitrary vectors. */
int tg_inverse_cdf(const float *p_host, int n, float cum0, float randf, int *idx, float *cum_out);
/* ops::rmsnorm, ops.hpp:182-222, rows x dim in place */
int tg_rmsnorm(float *x_host, const float *w_host, int rows, int dim);

/* ---- device-pointer variants (data already in HBM; used for kernel timing) */
int tg_dev_qmatvec(float *y_dev, const float *x_dev, const int8_t *w_dev, const float *scales_dev, int K, int N,
                   void *cuda_stream);
/* Same operator as tg_dev_qmatvec for callers that must not allocate device memory when they
 * call it: processes that hand all of HBM to their own pools, latency-critical loops that cannot
 * afford the allocator's implicit synchronisation, code running under stream capture. It has no
 * counterpart in the reference. The split-K partial sums and tile tickets live in a fixed
 * 264 KiB array inside the library (held by every GPU that loads it until exit) instead of
 * buffers grown with cudaMalloc; the call makes no cudaMalloc / cudaFree. Limits: N <= 262144
 * and nsplit * N <= 65536 partial sums (the split is chosen to fit); larger sizes are rejected
 * with TG_EINVAL. The first call on a device looks up the array's device address (with that
 * device current) and should therefore be made before any stream capture. All calls share the
 * array — it is cleared where it must start at zero — so two calls that overlap on the GPU
 * (different streams) race; serialise them. */
int tg_dev_qmatvec_static(float *y_dev, const float *x_dev, const int8_t *w_dev, const float *scales_dev, int K, int N,
                          void *cuda_stream);
/* tg_dev_qgemm synchronises the stream before it returns (it reads the kernel's error word), except
 * while the stream is being captured into a CUDA graph: then it only records its launches, and an
 * error raised by a replay is reported by the next call made outside a capture. */
int tg_dev_qgemm(float *c_dev, const float *a_dev, const int8_t *w_dev, const float *scales_dev, int M, int K, int N,
                 void *cuda_stream);

/* ---- vocab-sharded lm_head (multi-GPU variant) --------------------------- */
/* The reference scores the whole vocabulary in modules::lm_head (modules.hpp:223-247) and takes
 * the argmax (ops.hpp:744). With the [D, V] lm_head split by columns over several GPUs, each GPU
 * (1) runs the layers for its own sequences and stops before the lm_head (tg_decode_hidden; the
 * final-normed hidden states stay in HBM, tg_dev_hidden_copy copies them out [batch, D]),
 * (2) after the hidden states of all GPUs have been gathered, scores M of them against its own
 * column slice [col0, col0 + ncols) and returns per row the maximum logit and its global index,
 * lowest index on ties (tg_dev_lm_head_top1), and (3) after the per-slice candidates have been
 * gathered, resolves them (tg_dev_resolve_top1: largest maximum, lowest index among equal maxima,
 * ops.hpp:744-760) and takes the tokens of its own sequences back (tg_dev_set_tokens). The two
 * gathers are the caller's (NCCL). col0 and ncols must be multiples of 128.
 *
 * A step enqueues only: tg_decode_hidden with ids_host == NULL (tokens fed from the device),
 * tg_dev_hidden_copy, tg_dev_set_tokens (all on the state's stream) and tg_dev_lm_head_top1 /
 * tg_dev_resolve_top1 (on the stream given) never synchronise the host; enqueue everything of a
 * step on the state's stream (tg_state_stream). tg_state_check synchronises that stream and reports
 * the kernels' error word (bad token id, cache full, a wait that ran out); tg_decode_hidden with
 * host ids does the same before it returns. tg_dev_lm_head_top1 is one tensor-core GEMM over the
 * slice whose epilogue keeps the row maxima (no logits are written); a pipeline wait that ran out
 * in it is reported by the next call on the same device.
 * tg_dev_resolve_top1: cand_all_dev is [world][2][M] 32-bit words, per slice the M maxima (fp32)
 * then the M global indices (int32, -1: no candidate); writes the tokens of rows row0..row0+nrows. */
int tg_decode_hidden(tg_state *s, const int *ids_host);
int tg_state_check(tg_state *s);
int tg_dev_hidden_copy(tg_state *s, float *dst_dev);
int tg_dev_lm_head_top1(tg_model *m, const float *hidden_dev, int M, int col0, int ncols, float *max_dev, int *idx_dev,
                        void *cuda_stream);
int tg_dev_resolve_top1(const void *cand_all_dev, int world, int M, int row0, int nrows, int *toks_dev, void *cuda_stream);
int tg_dev_set_tokens(tg_state *s, const int *toks_dev);

/* ---- introspection for benchmarks --------------------------------------- */
/* number of kernels this library launched since the last call with reset != 0 */
int tg_launch_count(int reset, long long *count);
/* cudaStream_t the state launches on (as void*), for event timing by the caller */
int tg_state_stream(tg_state *s, void **cuda_stream);
/* enqueue n_steps of decode + greedy/min-p sampling on the state's stream and
 * return without synchronising (tokens stay on the device); pair with
 * tg_state_stream + events to time the device-resident loop. */
int tg_generate_async(tg_state *s, int n_steps, float minp, float temp);
/* upload uniforms [n, batch] used by min-p steps of tg_generate_async */
int tg_state_set_randf(tg_state *s, const float *randf_host, int n);
/* profiling aid for the persistent decode kernel: the first call arms a recorder;
 * afterwards each launch stores SM-clock stamps taken by CTA 0 at the phase
 * boundaries of its last token, and this call returns them (n = count). */
int tg_state_phase_clocks(tg_state *s, long long *clocks_host, int cap, int *n);
/* copy out the tokens the last tg_generate_async produced: [n_steps, batch] */
int tg_state_tokens(tg_state *s, int n_steps, int *toks_host);

#ifdef __cplusplus
}
#endif
#endif /* TINY_GEMMA_B200_H */
