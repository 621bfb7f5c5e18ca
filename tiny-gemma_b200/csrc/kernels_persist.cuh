// Persistent decode kernel: the whole per-token forward (and the sampler) of one
// sequence in ONE cooperative launch, one CTA per SM, 12 warps per CTA.
//
// At batch 1 a Gemma-3-1B layer is 26.8 MB of int8 weights — 4 us of HBM time —
// spread over five dependent phases, so the time of a token is the length of
// that dependency chain, not the data movement. The design therefore
//   * streams weights a layer ahead: every CTA owns a fixed unit of each weight
//     matrix (column groups x K-range), stored contiguously in a re-tiled copy,
//     and fetches it with bulk copies (cp.async.bulk) into a shared-memory
//     region reserved for that phase. A region is refilled for the NEXT layer
//     as soon as its last reader is done, so about one layer of weights per SM
//     is always in flight and HBM never waits for the chain;
//   * makes the tile products warp-autonomous. The activation vector is
//     quantised once per phase to 24-bit block fixed point (three 8-bit digit
//     planes, one power-of-two exponent per vector), the weight unit is stored
//     as 16-byte pieces of 4 rows x 4 columns (a 32-bit word = 4 consecutive
//     rows of one column), and a lane accumulates dp4a(word, digit plane) for
//     its 4 columns: the products and sums are exact integers, there is no
//     int8 -> fp32 conversion in the loop, and a warp finishes its own columns
//     with six shuffles — no block-wide barrier in any product;
//   * hands results over through small L2-resident vectors that validate
//     themselves (a sentinel marks words not yet written). Polled bytes are the
//     cost of a hand-off (about 40 ns per KB and CTA), so producers publish
//     final, scaled values wherever a consumer would otherwise re-add K-split
//     partial sums;
//   * recomputes RMSNorms redundantly in every CTA from those vectors; the
//     residual stream lives in each CTA's shared memory.
//
// Phases per layer (reference modules.hpp:135-169, 203-220):
//   A  residual + post-norm of the previous MLP, pre-norm, Q|K|V  -> q|k|v
//   B  q/k norm, RoPE, KV append, attention: CTA = (head, chunk of the cache)
//                                                    -> (m, l, o) per chunk
//   C  merge of the chunks of one head, O projection -> partial sums per head
//   D  residual + post-norm, pre-norm, up & gate, LUT-GeGLU -> activations
//   E  down projection                               -> partial sums per split
// then the lm_head (streamed through a ring of bulk copies from a re-tiled
// copy) and the sampler (argmax, or min-p with the sequential fp32 inverse CDF
// of reference ops.hpp:848-858 evaluated by an exact scan).
//
// Arithmetic: y[n] = scale[n] * sum_k x[k] W[k,n] (reference linalg.hpp:41-204)
// with x rounded to 24 significant bits relative to the largest |x| of the
// vector (fp32 itself keeps 24 bits relative to each element); products and
// sums are exact, one rounding when the integer sum becomes a float.
//
// Every wait is bounded: a spin that runs out sets *err and a shared abort
// flag, after which all waits fall through and the kernel returns.
#pragma once
#include <cuda.h>

#include "kernels_decode.cuh"
#include "kernels_sampler.cuh"
#include "tg_common.cuh"

namespace tg {

constexpr int PS_THREADS = 384;
constexpr int PS_NW = PS_THREADS / 32;
constexpr int PS_MAX_LAYERS = 32;
constexpr int PS_MAX_CH = 32;            // most cache chunks per head
constexpr int PS_ATT_ROW = AT_HD + 8;    // floats per attention partial: o[256], m, l, padding
constexpr int PS_SAMP_TILE = 128;        // vocabulary tile of the sampler's passes (same partition as minp_grid_kernel)
constexpr uint32_t PS_BULK_PIECE = 16384;
constexpr unsigned PS_EMPTY = 0xFFFFFFFFu;  // "not written yet": a NaN no computation produces

struct PsPhase {
	int ngroups;  // column groups (4 columns each) of a unit, per matrix
	int nq;       // quads (4 rows each) of a unit
	int nsplit;   // K-splits across CTAs
	int ntiles;   // column tiles
	int units;    // ntiles * nsplit
	int kp;       // warps that share one column group (they split its quads)
	int wq;       // quads per warp
	int bytes;    // bytes of a unit
	int cta0;     // CTA of unit 0
};

struct PsLayer {
	const float *sq, *sk, *sv, *so, *su, *sg, *sd;  // per-column scales
	const float *rmsq, *rmsk, *attn_pre, *attn_post, *mlp_pre, *mlp_post;
	float *kcache, *vcache;
	int slots, is_local;
};

struct PsArgs {
	const int8_t *tiled;  // re-tiled layer weights: per layer [A units | C units | D units (up, gate) | E units]
	size_t tl_layer, tl_A, tl_C, tl_D, tl_E;
	const int8_t *lm_tiled;  // re-tiled lm_head: [tile][chunk][group][quad] pieces
	const PsLayer *layers;
	int L, D, I, V, QD, KD;
	PsPhase A, C, Dp, E;
	// lm_head: column tiles of lm_groups * 4 columns; a tile's rows arrive as lm_nchunk ring stages of lm_cq quads
	int lm_groups, lm_cq, lm_nchunk, lm_ntiles, lm_stages, lm_stage_bytes;
	const float *lm_scale, *final_norm;
	const int8_t *wte;
	const float *wte_s;
	float sqrtD;
	const float *rope[2][2];  // [is_local][cos, sin]
	GeluLut lut;
	int off_A, off_C, off_D, off_E, off_h, off_xd, off_att, smem_total;
	int xd_words;  // words per digit plane buffer
	// Hand-off arena, three copies used by consecutive layers; every float is PS_EMPTY or a value.
	//   ll_qkv [QD + 2 KD]                 q|k|v, scaled                      (A -> B)
	//   ll_att [4][PS_MAX_CH][PS_ATT_ROW]  attention partials per head, chunk (B -> C)
	//   ll_op  [C.nsplit][D]               O projection, scaled partial sums  (C -> D)
	//   ll_act [I]                         GeGLU activations                  (D -> E)
	//   ll_dn  [E.nsplit][D] + presence    down projection, scaled partials   (E -> A of the next layer);
	//                                      one presence word for every CTA without a down unit
	float *ll;
	int ll_stride, ll_qkv, ll_att, ll_op, ll_act, ll_dn, ll_pres;
	int nch_local, nch_mid, nch_long;  // cache chunks per head: sliding-window layers / global up to 2048 keys / beyond
	float *logits;
	float *probs;
	int samp_ch;
	float *samp_f;
	int *samp_i;
	float *xnorm_out;
	unsigned *bar;          // grid-barrier counter: bar_base arrivals so far (it is never reset between launches)
	unsigned bar_base;
	int *err;
	int *tok, *next_pos, *ring_base, *tok_log, *log_count;
	int log_cap, n_steps, sampler;
	const int *force_ids;  // optional [n_steps]: the token of every step is given (continuation of a context), not sampled
	float minp, temp;
	const float *randf;
	int *randf_count;
	int randf_cap;
	long long *dbg;
	int dbg_cta, dbg_cap;
	long long wait_clocks;  // SM clocks before a wait gives up
	int poll_ns;            // sleep between two rounds of a hand-off poll
	int sched;              // 0: up/gate and down units of layer l+1 requested in phase E of layer l; 1: units of layer l requested after the Q|K|V product of layer l
	long long *gt;  // optional: [CTA][12] global-timer marks of one layer (DBG instantiation)
	int *beacon;    // optional (mapped host memory): [CTA][16] progress marks of every warp, for diagnosing a stall
	int e_rows;     // 1: the down projection runs by K-parts per warp (ps_product_rows), e_wq quads per warp
	int e_wq;
	int fault_cta;  // test hook: this CTA withholds its down-projection hand-off (-1: none); the waits then run out
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t ps_smem(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ps_mbar_init(uint64_t *bar, int count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ps_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ps_mbar_expect(uint64_t *bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ps_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ps_mbar_arrive(uint64_t *bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ps_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ps_mbar_try(uint64_t *bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok)
	    : "r"(ps_smem(bar)), "r"(parity)
	    : "memory");
	return ok != 0;
}
// Weights are read once per token: evict-first keeps the L2 for the KV cache and the hand-off vectors.
__device__ __forceinline__ uint64_t ps_evict_first() {
	uint64_t pol;
	asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
	return pol;
}
// Untiled bulk copy global -> this CTA's shared memory, completing on an mbarrier (never cluster-wide).
__device__ __forceinline__ void ps_bulk(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
	asm volatile(
	    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(ps_smem(dst)),
	    "l"(src), "r"(bytes), "r"(ps_smem(bar)), "l"(pol)
	    : "memory");
}
// Small vectors that every token reads again (column scales, norm weights, RoPE rows): kept in the L2
// (evict-last) so that they are L2 hits while the weight stream (evict-first) passes through.
__device__ __forceinline__ uint64_t ps_evict_last() {
	uint64_t pol;
	asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
	return pol;
}
__device__ __forceinline__ float ps_ldk(const float *p, uint64_t keep) {
	float v;
	asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(keep));
	return v;
}
__device__ __forceinline__ float4 ps_ldk4(const float *p, uint64_t keep) {
	float4 v;
	asm volatile("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(keep));
	return v;
}
__device__ __forceinline__ void ps_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void ps_prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ unsigned ps_ld_acquire(const unsigned *p) {
	unsigned v;
	asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}
__device__ __forceinline__ void ps_st(float *p, float v) { asm volatile("st.relaxed.gpu.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory"); }
__device__ __forceinline__ float4 ps_ld4(const float *p) {
	float4 r;
	asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p) : "memory");
	return r;
}
__device__ __forceinline__ float2 ps_ld2(const float *p) {
	float2 r;
	asm volatile("ld.relaxed.gpu.global.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "l"(p) : "memory");
	return r;
}
__device__ __forceinline__ float ps_ld1(const float *p) {
	float r;
	asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(r) : "l"(p) : "memory");
	return r;
}
__device__ __forceinline__ bool ps_ok(float v) { return __float_as_uint(v) != PS_EMPTY; }
__device__ __forceinline__ bool ps_ok(const float2 &v) { return ps_ok(v.x) && ps_ok(v.y); }
__device__ __forceinline__ bool ps_ok(const float4 &v) { return ps_ok(v.x) && ps_ok(v.y) && ps_ok(v.z) && ps_ok(v.w); }
__device__ __forceinline__ int ps_dp4a_su(uint32_t a, uint32_t b, int c) {  // signed bytes of a times unsigned bytes of b
	int d;
	asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
	return d;
}
__device__ __forceinline__ int ps_dp4a_ss(uint32_t a, uint32_t b, int c) {
	int d;
	asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
	return d;
}

// What a wait needs to know to give up: the CTA's abort flag, the global error word, the time limit.
struct PsW {
	int *s_abort;
	int *err;
	long long limit;  // SM clocks a wait may take
	unsigned nap;     // nanoseconds a poller sleeps between rounds
};
__device__ __forceinline__ bool ps_mbar_test(uint64_t *bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok)
	    : "r"(ps_smem(bar)), "r"(parity)
	    : "memory");
	return ok != 0;
}
// Give up: the first error code wins (code in the low byte, `where` = layer << 4 | phase above it);
// every later wait of this CTA falls through.
__device__ __noinline__ void ps_give_up(int *s_abort, int *err, int code) {
	*s_abort = 1;
	atomicCAS(err, 0, code);
}
// Wait for a bulk-copy barrier: non-blocking test in a loop bounded by the clock (the blocking
// try_wait form may suspend a thread for an unspecified time per call).
__device__ __noinline__ void ps_wait_bulk_slow(const PsW w, int where, uint64_t *bar, uint32_t parity) {
	const long long t0 = clock64();
	int spins = 0;
	while (!ps_mbar_test(bar, parity)) {
		if ((++spins & 63) == 0 && (clock64() - t0 > w.limit || *(volatile int *)w.s_abort)) {
			ps_give_up(w.s_abort, w.err, 3 | (where << 8));
			return;
		}
	}
}
__device__ __forceinline__ void ps_wait_bulk(const PsW &w, int where, uint64_t *bar, uint32_t parity) {
	if (*(volatile int *)w.s_abort) return;
	if (!ps_mbar_test(bar, parity)) ps_wait_bulk_slow(w, where, bar, parity);
}
// One more round of a hand-off poll? Gives up when the wait has taken w.limit clocks; a CTA that
// gave up (or saw the global error word) lets every later wait fall through.
__device__ __noinline__ bool ps_retry_slow(const PsW w, int where, long long t0) {
	if (clock64() - t0 > w.limit || *(volatile int *)w.err != 0) {
		ps_give_up(w.s_abort, w.err, 5 | (where << 8));
		return false;
	}
	return true;
}
__device__ __forceinline__ bool ps_retry(const PsW &w, int where, int &spins, long long &t0) {
	if (*(volatile int *)w.s_abort) return false;
	if (spins == 0) t0 = clock64();
	if ((++spins & 15) == 0 && !ps_retry_slow(w, where, t0)) return false;
	__nanosleep(w.nap);
	return true;
}

// grid-wide barrier: one atomic counter, bounded spin
__device__ __noinline__ void ps_grid_sync(const PsW w, int where, unsigned *bar, unsigned target) {
	__syncthreads();
	if (threadIdx.x == 0) {
		__threadfence();
		const unsigned old = atomicAdd(bar, 1u);
		// (the counter runs on from launch to launch and may wrap: compare differences, not values)
		if (old + 1u != target && !*(volatile int *)w.s_abort) {  // the last arriver need not poll
			const long long t0 = clock64();
			int spins = 0;
			while (int(ps_ld_acquire(bar) - target) < 0) {
				if ((++spins & 15) == 0 && clock64() - t0 > w.limit) {
					ps_give_up(w.s_abort, w.err, 4 | (where << 8));
					break;
				}
			}
		}
	}
	__syncthreads();
}

// ------------------------------------------------------------------ quantised activations
// A vector x[0..4 nq) becomes three word planes xd[p * stride + q], p = 0, 1, 2: byte j of word q of plane p is
// digit p of round(x[4q + j] * 2^(23 - e)), digits 0 and 1 unsigned, digit 2 signed, where 2^e > max |x|.
// ps_exponent returns e for a bound on max |x| (clamped so that both scale factors are normal floats).
__device__ __forceinline__ int ps_exponent(float bound) {
	const int eb = int(__float_as_uint(bound) >> 23) & 0xFF;  // bound in [2^(eb-127), 2^(eb-126))
	return max(-100, min(100, eb - 126));
}
__device__ __forceinline__ float ps_pow2(int e) { return __uint_as_float(uint32_t(e + 127) << 23); }
__device__ __forceinline__ void ps_quantise(float4 y, float qs, uint32_t *xd, int stride, int q) {
	__builtin_assume(__isShared(xd));
	int v[4];
	v[0] = __float2int_rn(y.x * qs);
	v[1] = __float2int_rn(y.y * qs);
	v[2] = __float2int_rn(y.z * qs);
	v[3] = __float2int_rn(y.w * qs);
#pragma unroll
	for (int i = 0; i < 4; i++) v[i] = max(-8388607, min(8388607, v[i]));
	const uint32_t p01 = __byte_perm(v[0], v[1], 0x5140), p23 = __byte_perm(v[2], v[3], 0x5140);
	const uint32_t h01 = __byte_perm(v[0], v[1], 0x0062), h23 = __byte_perm(v[2], v[3], 0x0062);
	xd[q] = __byte_perm(p01, p23, 0x5410);
	xd[stride + q] = __byte_perm(p01, p23, 0x7632);
	xd[2 * stride + q] = __byte_perm(h01, h23, 0x5410);
}
// max over the CTA of a non-negative value through `red` (12 floats; one barrier), then the exponent for it
__device__ __forceinline__ int ps_block_exponent(float mx, float *red) {
	mx = warp_max(mx);
	if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
	__syncthreads();
	float M = 0.0f;
#pragma unroll
	for (int w = 0; w < PS_NW; w++) M = fmaxf(M, red[w]);
	return ps_exponent(M * 1.000001f);
}

// ------------------------------------------------------------------ tile products
// piece (group g, quad q) of a unit sits at tile[g * nq + q]; word c of a piece = column 4g + c, its
// bytes = rows 4q .. 4q+3. acc[3c + p] += dp4a(word c, digit plane p).
struct PsAcc {
	int v[12];
};
__device__ __forceinline__ void ps_mac(PsAcc &a, const uint4 &w, uint32_t x0, uint32_t x1, uint32_t x2) {
	const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
	for (int c = 0; c < 4; c++) {
		a.v[3 * c] = ps_dp4a_su(ww[c], x0, a.v[3 * c]);
		a.v[3 * c + 1] = ps_dp4a_su(ww[c], x1, a.v[3 * c + 1]);
		a.v[3 * c + 2] = ps_dp4a_ss(ww[c], x2, a.v[3 * c + 2]);
	}
}
// Lane sums of one group -> warp sums. The three digit sums of a column combine to
// S = a2 * 65536 + a1 * 256 + a0 in fp32 (each below 2^22 per lane: exact conversions, one rounding
// per fma), then the four columns are reduced over the lanes by halving (2 + 1 + 1 + 1 + 1
// shuffles). Lanes 0..3 return the sum of column `lane`. Called by whole warps.
__device__ __noinline__ float ps_finish(const PsAcc a) {
	const int lane = threadIdx.x & 31;
	float v[4];
#pragma unroll
	for (int c = 0; c < 4; c++) {
		// |digit sum| < 2^22 (at most 32 quads per lane: 32 * 4 * 127 * 255): exact int -> float through the
		// mantissa of 1.5 * 2^23, one add and one subtract instead of a conversion instruction
		const float f0 = __int_as_float(0x4B400000 + a.v[3 * c]) - 12582912.0f;
		const float f1 = __int_as_float(0x4B400000 + a.v[3 * c + 1]) - 12582912.0f;
		const float f2 = __int_as_float(0x4B400000 + a.v[3 * c + 2]) - 12582912.0f;
		v[c] = fmaf(f2, 65536.0f, fmaf(f1, 256.0f, f0));
	}
	{
		const bool up = lane & 16;
		const float s0 = up ? v[0] : v[2], s1 = up ? v[1] : v[3];
		const float k0 = up ? v[2] : v[0], k1 = up ? v[3] : v[1];
		v[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 16);
		v[1] = k1 + __shfl_xor_sync(0xffffffffu, s1, 16);
	}
	{
		const bool up = lane & 8;
		const float s = up ? v[0] : v[1], k = up ? v[1] : v[0];
		v[0] = k + __shfl_xor_sync(0xffffffffu, s, 8);
	}
	v[0] += __shfl_xor_sync(0xffffffffu, v[0], 4);
	v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
	v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
	// lane 8 * (2 b4 + b3) holds column 2 b4 + b3
	return __shfl_sync(0xffffffffu, v[0], (lane & 3) * 8);
}
// Shared-memory accesses by 32-bit shared-window address. The helpers below are not inlined (code
// size), so a pointer argument would be a generic pointer and every access a generic load, which
// runs at about half the rate of ld.shared in the product loop.
__device__ __forceinline__ uint4 ps_lds128(uint32_t addr) {
	uint4 v;
	asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
	return v;
}
__device__ __forceinline__ uint32_t ps_lds32(uint32_t addr) {
	uint32_t v;
	asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
	return v;
}
__device__ __forceinline__ float ps_ldsf(uint32_t addr) {
	float v;
	asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
	return v;
}
__device__ __forceinline__ void ps_stsf(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
// Two groups at once: the two reductions' shuffles overlap. Lanes 0..3: (r0, r1) of column `lane`.
__device__ __noinline__ float2 ps_finish2(const PsAcc a, const PsAcc b) {
	const int lane = threadIdx.x & 31;
	float v[4], u[4];
#pragma unroll
	for (int c = 0; c < 4; c++) {
		const float f0 = __int_as_float(0x4B400000 + a.v[3 * c]) - 12582912.0f;
		const float f1 = __int_as_float(0x4B400000 + a.v[3 * c + 1]) - 12582912.0f;
		const float f2 = __int_as_float(0x4B400000 + a.v[3 * c + 2]) - 12582912.0f;
		v[c] = fmaf(f2, 65536.0f, fmaf(f1, 256.0f, f0));
		const float g0 = __int_as_float(0x4B400000 + b.v[3 * c]) - 12582912.0f;
		const float g1 = __int_as_float(0x4B400000 + b.v[3 * c + 1]) - 12582912.0f;
		const float g2 = __int_as_float(0x4B400000 + b.v[3 * c + 2]) - 12582912.0f;
		u[c] = fmaf(g2, 65536.0f, fmaf(g1, 256.0f, g0));
	}
	{
		const bool up = lane & 16;
		const float s0 = up ? v[0] : v[2], s1 = up ? v[1] : v[3], t0 = up ? u[0] : u[2], t1 = up ? u[1] : u[3];
		const float k0 = up ? v[2] : v[0], k1 = up ? v[3] : v[1], m0 = up ? u[2] : u[0], m1 = up ? u[3] : u[1];
		v[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 16);
		v[1] = k1 + __shfl_xor_sync(0xffffffffu, s1, 16);
		u[0] = m0 + __shfl_xor_sync(0xffffffffu, t0, 16);
		u[1] = m1 + __shfl_xor_sync(0xffffffffu, t1, 16);
	}
	{
		const bool up = lane & 8;
		const float s = up ? v[0] : v[1], k = up ? v[1] : v[0], t = up ? u[0] : u[1], m = up ? u[1] : u[0];
		v[0] = k + __shfl_xor_sync(0xffffffffu, s, 8);
		u[0] = m + __shfl_xor_sync(0xffffffffu, t, 8);
	}
#pragma unroll
	for (int o = 4; o > 0; o >>= 1) {
		v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
		u[0] += __shfl_xor_sync(0xffffffffu, u[0], o);
	}
	return make_float2(__shfl_sync(0xffffffffu, v[0], (lane & 3) * 8), __shfl_sync(0xffffffffu, u[0], (lane & 3) * 8));
}
// The warp that completes a count: every warp calls this once per round after its work; the one
// that makes the count reach `total` gets true (and resets the counter for the next round).
__device__ __forceinline__ bool ps_last(uint32_t cnt_s, int total) {
	const int lane = threadIdx.x & 31;
	__syncwarp();
	int old = 0;
	if (lane == 0) {
		__threadfence_block();
		asm volatile("atom.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(cnt_s) : "memory");
		if (old == total - 1) asm volatile("st.shared.u32 [%0], %1;" ::"r"(cnt_s), "r"(0) : "memory");
	}
	old = __shfl_sync(0xffffffffu, old, 0);
	if (old == total - 1) __threadfence_block();  // the other warps' shared-memory writes are visible to every lane
	return old == total - 1;
}
// Column sums of one unit: warp -> (group = warp / kp, part = warp % kp) takes quads part * wq .. of
// its group, of one matrix or of two matrices of the same shape that share the activations (up, then
// gate: `two`). tile_s, xd_s, part_s (PS_NW * 8 floats), cnt_s (PS_NW + 1 ints) are shared-window
// addresses. flags bit 0: this warp publishes its group (it is the only warp of the group, or the last
// of its kp warps to finish, and has added the parts in part order): lanes 0..3 hold the raw sums of
// columns 4 * group + lane in r0 (and r1). Bit 1: nobody reads the tile any more after this warp.
struct PsOut {
	float r0, r1;
	int flags;
};
// what a CTA's place in the grid fixes for the whole launch (kept in shared memory, read where it is used)
struct PsCta {
	const int8_t *srcA, *srcC, *srcD, *srcE;
	int tileA, tileC, splitC, tileE, splitE, presE, uD, has;
};
__device__ __noinline__ PsOut ps_product(uint32_t tile_s, int ngroups, int nq, int kp, int wq, bool two, uint32_t xd_s, int xs,
                                         uint32_t part_s, uint32_t cnt_s, long long *trace = nullptr) {
	PsOut o{0.0f, 0.0f, 0};
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	if (trace && lane == 0) trace[warp * 4] = clock64();
	const int group = warp / kp;
	if (group >= ngroups) return o;
	const int part = warp - group * kp;
	const int q1 = min(nq, (part + 1) * wq);
	PsAcc a0, a1;
#pragma unroll
	for (int i = 0; i < 12; i++) a0.v[i] = a1.v[i] = 0;
	const uint32_t t0 = tile_s + uint32_t(group * nq) * 16u, t1 = tile_s + uint32_t((ngroups + group) * nq) * 16u;
	int q = part * wq + lane;
	// two quads per round: the second quad's loads are in flight while the first one's products issue
	// (requesting the next round's operands a round ahead was measured slower: more registers, no gain)
#pragma unroll 1
	for (; q + 32 < q1; q += 64) {
		const uint32_t xa = xd_s + 4u * q;
		const uint32_t x0 = ps_lds32(xa), x1 = ps_lds32(xa + 4u * xs), x2 = ps_lds32(xa + 8u * xs);
		const uint32_t y0 = ps_lds32(xa + 128u), y1 = ps_lds32(xa + 4u * xs + 128u), y2 = ps_lds32(xa + 8u * xs + 128u);
		const uint4 w0 = ps_lds128(t0 + 16u * q), w1 = ps_lds128(t0 + 16u * q + 512u);
		if (two) {
			const uint4 v0 = ps_lds128(t1 + 16u * q), v1 = ps_lds128(t1 + 16u * q + 512u);
			ps_mac(a1, v0, x0, x1, x2);
			ps_mac(a1, v1, y0, y1, y2);
		}
		ps_mac(a0, w0, x0, x1, x2);
		ps_mac(a0, w1, y0, y1, y2);
	}
#pragma unroll 1
	for (; q < q1; q += 32) {
		const uint32_t xa = xd_s + 4u * q;
		const uint32_t x0 = ps_lds32(xa), x1 = ps_lds32(xa + 4u * xs), x2 = ps_lds32(xa + 8u * xs);
		ps_mac(a0, ps_lds128(t0 + 16u * q), x0, x1, x2);
		if (two) ps_mac(a1, ps_lds128(t1 + 16u * q), x0, x1, x2);
	}
	if (trace && lane == 0) trace[warp * 4 + 1] = clock64();
	if (two) {
		const float2 r = ps_finish2(a0, a1);
		o.r0 = r.x;
		o.r1 = r.y;
	} else {
		o.r0 = ps_finish(a0);
	}
	if (trace && lane == 0) trace[warp * 4 + 2] = clock64();
	bool pub = true;
	if (kp > 1) {
		if (lane < 4) {
			ps_stsf(part_s + 4u * (warp * 8 + lane), o.r0);
			ps_stsf(part_s + 4u * (warp * 8 + 4 + lane), o.r1);
		}
		pub = ps_last(cnt_s + 4u * (1 + group), kp);
		if (pub) {
			o.r0 = o.r1 = 0.0f;
			if (lane < 4)
				for (int p = 0; p < kp; p++) {
					o.r0 += ps_ldsf(part_s + 4u * ((group * kp + p) * 8 + lane));
					o.r1 += ps_ldsf(part_s + 4u * ((group * kp + p) * 8 + 4 + lane));
				}
		}
	}
	if (pub) o.flags = 1 | (ps_last(cnt_s, ngroups) ? 2 : 0);
	if (trace && lane == 0) trace[warp * 4 + 3] = clock64();
	return o;
}

// Down projection without a CTA-wide prologue. Warp w takes K-part w of the unit (quads w * wq .. of every
// group; lane -> quads lane, lane + 32, lane + 64 of the part, wq <= 96): it polls ITS rows of the activation
// vector, quantises them with a warp-local exponent into registers, multiplies them with all ngroups <= 4
// groups of the tile and leaves scaled fp32 partial sums in part_s[w][16]. The warp that finishes last adds
// the PS_NW parts in part order: its lanes 0 .. 4 * ngroups - 1 return the raw sums of columns
// 4 * group + (lane & 3), group = lane / 4, in r0, with flags = 3. No warp waits for another warp's rows, so
// a late producer delays only the part that needs it. part_s: PS_NW * 16 floats; cnt_s: one counter.
__device__ __noinline__ PsOut ps_product_rows(const PsW w, int where, uint32_t tile_s, int ngroups, int nq, int wq, const float *act,
                                              uint32_t part_s, uint32_t cnt_s, long long *trace = nullptr) {
	PsOut o{0.0f, 0.0f, 0};
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	if (trace && lane == 0) trace[warp * 4] = clock64();
	const int qb = warp * wq, qe = min(nq, qb + wq);  // this warp's quads
	float4 v[3];
	{
		int spins = 0;
		long long t0 = 0;
		bool ok;
		do {
			ok = true;
#pragma unroll
			for (int i = 0; i < 3; i++) {
				const int q = qb + lane + 32 * i;
				v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
				if (q < qe) v[i] = ps_ld4(act + 4 * q);
				ok = ok && ps_ok(v[i]);
			}
		} while (!ok && ps_retry(w, where, spins, t0));
	}
	float mx = 0.0f;
#pragma unroll
	for (int i = 0; i < 3; i++) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
	mx = warp_max(mx);
	if (trace && lane == 0) trace[warp * 4 + 1] = clock64();
	const int e = ps_exponent(mx * 1.000001f);
	const float qs = ps_pow2(23 - e), back = ps_pow2(e - 23);
	uint32_t x0[3], x1[3], x2[3];
#pragma unroll
	for (int i = 0; i < 3; i++) {
		int d[4];
		d[0] = __float2int_rn(v[i].x * qs);
		d[1] = __float2int_rn(v[i].y * qs);
		d[2] = __float2int_rn(v[i].z * qs);
		d[3] = __float2int_rn(v[i].w * qs);
#pragma unroll
		for (int j = 0; j < 4; j++) d[j] = max(-8388607, min(8388607, d[j]));
		const uint32_t p01 = __byte_perm(d[0], d[1], 0x5140), p23 = __byte_perm(d[2], d[3], 0x5140);
		const uint32_t h01 = __byte_perm(d[0], d[1], 0x0062), h23 = __byte_perm(d[2], d[3], 0x0062);
		x0[i] = __byte_perm(p01, p23, 0x5410);
		x1[i] = __byte_perm(p01, p23, 0x7632);
		x2[i] = __byte_perm(h01, h23, 0x5410);
	}
	// quads past the part multiply zeros; their tile address is clamped into the part
	uint32_t ta[3];
#pragma unroll
	for (int i = 0; i < 3; i++) ta[i] = tile_s + 16u * uint32_t(min(qb + lane + 32 * i, qe - 1));
#pragma unroll 1
	for (int g = 0; g < ngroups; g += 2) {
		PsAcc a0, a1;
#pragma unroll
		for (int i = 0; i < 12; i++) a0.v[i] = a1.v[i] = 0;
		const uint32_t g0 = 16u * uint32_t(g * nq), g1 = 16u * uint32_t(min(g + 1, ngroups - 1) * nq);
#pragma unroll
		for (int i = 0; i < 3; i++) {
			ps_mac(a0, ps_lds128(ta[i] + g0), x0[i], x1[i], x2[i]);
			ps_mac(a1, ps_lds128(ta[i] + g1), x0[i], x1[i], x2[i]);
		}
		const float2 r = ps_finish2(a0, a1);
		if (lane < 4) {
			ps_stsf(part_s + 4u * (warp * 16 + 4 * g + lane), r.x * back);
			if (g + 1 < ngroups) ps_stsf(part_s + 4u * (warp * 16 + 4 * g + 4 + lane), r.y * back);
		}
	}
	if (trace && lane == 0) trace[warp * 4 + 2] = clock64();
	if (ps_last(cnt_s, PS_NW)) {
		o.flags = 3;
		if (lane < 4 * ngroups) {
#pragma unroll
			for (int p = 0; p < PS_NW; p++) o.r0 += ps_ldsf(part_s + 4u * (p * 16 + lane));
		}
	}
	if (trace && lane == 0) trace[warp * 4 + 3] = clock64();
	return o;
}

// A CTA's unit is one contiguous block of the re-tiled copy: one bulk copy. Called by one lane.
__device__ __noinline__ void ps_issue(uint8_t *dst, const int8_t *src, uint32_t bytes, uint64_t *bar, uint64_t pol, const int *abort_flag) {
	if (*(volatile const int *)abort_flag) return;  // a CTA that gave up starts no new copies
	// (no proxy fence: the region was only READ through the generic proxy, and those loads have completed —
	// their values were consumed before the readers signalled that the tile is free)
	ps_mbar_expect(bar, bytes);
	ps_bulk(dst, src, bytes, bar, pol);
}

// Re-tile `ntiles_mat` column tiles x `nsplit` K-splits of a row-major int8 matrix [K][N] into unit order:
// unit (split, tile0 + t) is a block at dst + (split * ntiles_total + tile0 + t) * unit_stride + dst_off
// holding the pieces [group][quad] of 16 bytes described at ps_dot. One thread per piece.
__device__ __forceinline__ uint4 ps_piece(const int8_t *src, size_t N, size_t row0, size_t col0) {
	const uint32_t r0 = *reinterpret_cast<const uint32_t *>(src + row0 * N + col0);
	const uint32_t r1 = *reinterpret_cast<const uint32_t *>(src + (row0 + 1) * N + col0);
	const uint32_t r2 = *reinterpret_cast<const uint32_t *>(src + (row0 + 2) * N + col0);
	const uint32_t r3 = *reinterpret_cast<const uint32_t *>(src + (row0 + 3) * N + col0);
	const uint32_t t0 = __byte_perm(r0, r1, 0x5140), t1 = __byte_perm(r2, r3, 0x5140);
	const uint32_t t2 = __byte_perm(r0, r1, 0x7362), t3 = __byte_perm(r2, r3, 0x7362);
	return make_uint4(__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632), __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632));
}
__global__ void retile_quads_kernel(int8_t *dst, const int8_t *src, int N, int ngroups, int nq, int nsplit, int ntiles_total,
                                    int tile0, int ntiles_mat, size_t unit_stride, size_t dst_off) {
	const size_t total = size_t(nsplit) * ntiles_mat * ngroups * nq;
	for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
		const int g = int(i % ngroups);
		const int t = int((i / ngroups) % ntiles_mat);
		const int q = int((i / (size_t(ngroups) * ntiles_mat)) % nq);
		const int split = int(i / (size_t(ngroups) * ntiles_mat * nq));
		const uint4 v = ps_piece(src, size_t(N), (size_t(split) * nq + q) * 4, (size_t(t) * ngroups + g) * 4);
		*reinterpret_cast<uint4 *>(dst + size_t(split * ntiles_total + tile0 + t) * unit_stride + dst_off + (size_t(g) * nq + q) * 16) = v;
	}
}
// lm_head [K][V] -> [tile][chunk][group][quad] pieces; columns past V (the last tile) are zero.
__global__ void retile_lm_kernel(int8_t *dst, const int8_t *src, int V, int ngroups, int cq, int nchunk, int ntiles) {
	const size_t gcols = size_t(ntiles) * ngroups;  // column groups in all
	const size_t total = gcols * cq * nchunk;
	for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
		const size_t gc = i % gcols;
		const int row_q = int(i / gcols);  // quad row of the whole matrix
		const int t = int(gc / ngroups), g = int(gc % ngroups);
		const int ch = row_q / cq, q = row_q % cq;
		uint4 v = make_uint4(0u, 0u, 0u, 0u);
		if (gc * 4 < size_t(V)) v = ps_piece(src, size_t(V), size_t(row_q) * 4, gc * 4);
		*reinterpret_cast<uint4 *>(dst + ((size_t(t) * nchunk + ch) * ngroups * cq + size_t(g) * cq + q) * 16) = v;
	}
}

// lut::GeLUTable::lookup (reference ops.hpp:41-51) with the table kept L2-resident
__device__ __forceinline__ float ps_gelu(const GeluLut &t, float x, uint64_t keep) {
	const float q = (x - t.mn) / t.eps;
	if (!(q < 2147483648.0f) || q < -2147483648.0f) return 0.0f;  // (x86 cvttss2si: INT_MIN, a negative index)
	const int idx = int(q);
	if (idx < 0) return 0.0f;
	if (idx >= t.size) return x;
	return ps_ldk(t.table + idx, keep);
}

// ------------------------------------------------------------------ prologues
// 1 / sqrt(sumsq / dim + eps): the hardware estimate refined by one Newton step, which is how the
// reference's build evaluates it (rsqrtss + one step under -ffast-math, reference ops.hpp:153)
__device__ __forceinline__ float ps_inv_rms(float sumsq, float inv_dim) {
	const float v = fmaf(sumsq, inv_dim, RMS_EPS);
	const float r = rsqrtf(v);
	return r * fmaf(-0.5f * v, r * r, 1.5f);
}
// If part: t[d] = sum_s part[s][d] (scaled partial sums, polled until complete; threads past D/4 poll
// the presence words);  h += rmsnorm(t; w_post). Then y = rmsnorm(h; w_pre), quantised into xd (stride
// D/4) with *s_xscale = 2^(e - 23). Every CTA computes the same bits. D <= 4 * PS_THREADS. Thread t
// owns elements 4t..4t+3, which are quad t. bred: 3 * PS_NW floats.
__device__ __noinline__ void ps_resnorm(const PsW w, int where, int D, float *h, uint32_t *xd, float *bred, float *s_xscale,
                                        const float *part, int nsplit, const float *pres, int npres, const float *w_post,
                                        const float *w_pre, uint64_t keep, float *x_out, long long *trace = nullptr) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	__builtin_assume(__isShared(h));
	__builtin_assume(__isShared(xd));
	__builtin_assume(__isShared(s_xscale));
	// the norm weights are L2-resident (evict-last): requested together with the first poll loads
	float4 wpost = make_float4(0.f, 0.f, 0.f, 0.f), wpre = wpost;
	if (4 * tid < D) {
		if (part) wpost = ps_ldk4(w_post + 4 * tid, keep);
		wpre = ps_ldk4(w_pre + 4 * tid, keep);
	}
	const uint32_t bred_s = ps_smem(bred);
	const float invD = 1.0f / float(D);
	if (trace && lane == 0) trace[warp * 5] = clock64();
	const bool in = 4 * tid < D;
	float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
	if (in) hv = *reinterpret_cast<const float4 *>(h + 4 * tid);
	if (part) {
		float4 tv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
		for (int s0 = 0; s0 < nsplit; s0 += 2) {
			float4 p0, p1;
			int spins = 0;
			long long t0 = 0;
			bool ok;
			do {
				p0 = p1 = make_float4(0.f, 0.f, 0.f, 0.f);
				if (in) {
					p0 = ps_ld4(part + size_t(s0) * D + 4 * tid);
					if (s0 + 1 < nsplit) p1 = ps_ld4(part + size_t(s0 + 1) * D + 4 * tid);
				}
				ok = ps_ok(p0) && ps_ok(p1);
				if (s0 == 0 && !in && tid - D / 4 < npres) ok = ps_ok(ps_ld1(pres + (tid - D / 4)));
			} while (!ok && ps_retry(w, where, spins, t0));
			tv.x += p0.x + p1.x;  // splits in ascending order (p1 is an exact zero when absent)
			tv.y += p0.y + p1.y;
			tv.z += p0.z + p1.z;
			tv.w += p0.w + p1.w;
		}
		if (trace && lane == 0) trace[warp * 5 + 1] = clock64();
		float ss = fmaf(tv.x, tv.x, fmaf(tv.y, tv.y, fmaf(tv.z, tv.z, tv.w * tv.w)));
		ss = warp_sum(ss);
		if (lane == 0) ps_stsf(bred_s + 4u * warp, ss);
		__syncthreads();
		if (trace && lane == 0) trace[warp * 5 + 2] = clock64();
		float t = 0.0f;
#pragma unroll
		for (int i = 0; i < PS_NW; i++) t += ps_ldsf(bred_s + 4u * i);
		const float r1 = ps_inv_rms(t, invD);
		hv.x = hv.x + (tv.x * r1) * (wpost.x + 1.0f);
		hv.y = hv.y + (tv.y * r1) * (wpost.y + 1.0f);
		hv.z = hv.z + (tv.z * r1) * (wpost.z + 1.0f);
		hv.w = hv.w + (tv.w * r1) * (wpost.w + 1.0f);
		if (in) *reinterpret_cast<float4 *>(h + 4 * tid) = hv;
	}
	const float4 g = make_float4(wpre.x + 1.0f, wpre.y + 1.0f, wpre.z + 1.0f, wpre.w + 1.0f);
	float ss2 = fmaf(hv.x, hv.x, fmaf(hv.y, hv.y, fmaf(hv.z, hv.z, hv.w * hv.w)));
	float mx = fmaxf(fmaxf(fabsf(hv.x * g.x), fabsf(hv.y * g.y)), fmaxf(fabsf(hv.z * g.z), fabsf(hv.w * g.w)));
	ss2 = warp_sum(ss2);
	mx = warp_max(mx);
	if (lane == 0) {
		ps_stsf(bred_s + 4u * (PS_NW + warp), ss2);
		ps_stsf(bred_s + 4u * (2 * PS_NW + warp), mx);
	}
	__syncthreads();
	if (trace && lane == 0) trace[warp * 5 + 3] = clock64();
	float t2 = 0.0f, m2 = 0.0f;
#pragma unroll
	for (int i = 0; i < PS_NW; i++) {
		t2 += ps_ldsf(bred_s + 4u * (PS_NW + i));
		m2 = fmaxf(m2, ps_ldsf(bred_s + 4u * (2 * PS_NW + i)));
	}
	const float r2 = ps_inv_rms(t2, invD);
	const int e = ps_exponent(r2 * m2 * 1.000001f);
	if (in) {
		float4 y;
		y.x = (hv.x * r2) * g.x;
		y.y = (hv.y * r2) * g.y;
		y.z = (hv.z * r2) * g.z;
		y.w = (hv.w * r2) * g.w;
		ps_quantise(y, ps_pow2(23 - e), xd, D / 4, tid);
		if (x_out) *reinterpret_cast<float4 *>(x_out + 4 * tid) = y;
	}
	if (tid == 0) *s_xscale = ps_pow2(e - 23);
	__syncthreads();
	if (trace && lane == 0) trace[warp * 5 + 4] = clock64();
}

// one warp: x[0..256) (dims 4 lane.. and 128 + 4 lane..) -> rmsnorm, RoPE, * scale -> dst (may alias x)
struct PsRope {
	float4 w0, w1, c0, c1, s0, s1;
};
__device__ __forceinline__ void ps_load_rope(PsRope &r, const float *w, const float *cosr, const float *sinr, uint64_t keep) {
	const int lane = threadIdx.x & 31;
	r.w0 = ps_ldk4(w + 4 * lane, keep);
	r.w1 = ps_ldk4(w + 128 + 4 * lane, keep);
	r.c0 = ps_ldk4(cosr + 4 * lane, keep);
	r.c1 = ps_ldk4(cosr + 128 + 4 * lane, keep);
	r.s0 = ps_ldk4(sinr + 4 * lane, keep);
	r.s1 = ps_ldk4(sinr + 128 + 4 * lane, keep);
}
__device__ __forceinline__ void ps_norm_rope(const float *x, const PsRope &r, float scale, float *dst) {
	const int lane = threadIdx.x & 31;
	const float4 lo4 = *reinterpret_cast<const float4 *>(x + 4 * lane), hi4 = *reinterpret_cast<const float4 *>(x + 128 + 4 * lane);
	const float lo[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hi[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
	const float w0[4] = {r.w0.x, r.w0.y, r.w0.z, r.w0.w}, w1[4] = {r.w1.x, r.w1.y, r.w1.z, r.w1.w};
	const float c0[4] = {r.c0.x, r.c0.y, r.c0.z, r.c0.w}, c1[4] = {r.c1.x, r.c1.y, r.c1.z, r.c1.w};
	const float s0[4] = {r.s0.x, r.s0.y, r.s0.z, r.s0.w}, s1[4] = {r.s1.x, r.s1.y, r.s1.z, r.s1.w};
	float ss = 0.0f;
#pragma unroll
	for (int i = 0; i < 4; i++) {
		ss = fmaf(lo[i], lo[i], ss);
		ss = fmaf(hi[i], hi[i], ss);
	}
	ss = warp_sum(ss);
	const float rr = inv_rms(ss, AT_HD);
	float ylo[4], yhi[4];
#pragma unroll
	for (int i = 0; i < 4; i++) {
		const float p = (lo[i] * rr) * (w0[i] + 1.0f);
		const float q = (hi[i] * rr) * (w1[i] + 1.0f);
		// y = cos * x + rotate_half(x) * sin, rotate_half = [-x_hi, x_lo] (reference decode.hpp:203-211)
		ylo[i] = fmaf(-1.0f * q, s0[i], c0[i] * p) * scale;
		yhi[i] = fmaf(p, s1[i], c1[i] * q) * scale;
	}
	__syncwarp();
	*reinterpret_cast<float4 *>(dst + 4 * lane) = make_float4(ylo[0], ylo[1], ylo[2], ylo[3]);
	*reinterpret_cast<float4 *>(dst + 128 + 4 * lane) = make_float4(yhi[0], yhi[1], yhi[2], yhi[3]);
}

// Phase C prologue: merge the attention partials of `hp` heads starting at head h0 over `nch` chunks
// into the normalised output (reference ops.hpp:316-357 keeps it normalised per step; the split form
// divides once), quantise it into xd (stride hp * 64).
__device__ __noinline__ void ps_attn_merge(const PsW w, int where, const float *att_ll, int h0, int hp, int nch, float *scr, uint32_t *xd,
                                           float *bred, float *s_xscale) {
	const int tid = threadIdx.x;
	__builtin_assume(__isShared(scr));
	__builtin_assume(__isShared(xd));
	__builtin_assume(__isShared(bred));
	__builtin_assume(__isShared(s_xscale));
	const int items = hp * (AT_HD / 4);  // float4 columns
	const int ncg = PS_THREADS / items;  // chunk groups
	const int cg = tid / items, it = tid - cg * items;
	const int hl = it / (AT_HD / 4), j = it - hl * (AT_HD / 4);
	float m = -INFINITY, l = 0.0f;
	float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
	if (cg < ncg) {
#pragma unroll 1
		for (int ch = cg; ch < nch; ch += ncg) {
			const float *r0 = att_ll + (size_t(h0 + hl) * PS_MAX_CH + ch) * PS_ATT_ROW;
			float4 ov;
			float2 ml;
			int spins = 0;
			long long t0 = 0;
			bool ok;
			do {
				ov = ps_ld4(r0 + 4 * j);
				ml = ps_ld2(r0 + AT_HD);
				ok = ps_ok(ov) && ps_ok(ml);
			} while (!ok && ps_retry(w, where, spins, t0));
			if (ml.x == -INFINITY) continue;  // empty chunk
			const float mn = fmaxf(m, ml.x);
			const float ea = expf(m - mn), eb = expf(ml.x - mn);
			l = fmaf(l, ea, ml.y * eb);
			o.x = fmaf(o.x, ea, ov.x * eb);
			o.y = fmaf(o.y, ea, ov.y * eb);
			o.z = fmaf(o.z, ea, ov.z * eb);
			o.w = fmaf(o.w, ea, ov.w * eb);
			m = mn;
		}
		float *s = scr + (size_t(cg) * items + it) * 8;
		*reinterpret_cast<float4 *>(s) = o;
		*reinterpret_cast<float2 *>(s + 4) = make_float2(m, l);
	}
	__syncthreads();
	float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
	float mx = 0.0f;
	if (tid < items) {
		float M = -INFINITY;
#pragma unroll 1
		for (int g = 0; g < ncg; g++) M = fmaxf(M, scr[(size_t(g) * items + tid) * 8 + 4]);
		float L = 0.0f;
#pragma unroll 1
		for (int g = 0; g < ncg; g++) {
			const float *s = scr + (size_t(g) * items + tid) * 8;
			const float mg = s[4];
			if (mg == -INFINITY) continue;
			const float e = expf(mg - M);
			const float4 ov = *reinterpret_cast<const float4 *>(s);
			L = fmaf(s[5], e, L);
			y.x = fmaf(ov.x, e, y.x);
			y.y = fmaf(ov.y, e, y.y);
			y.z = fmaf(ov.z, e, y.z);
			y.w = fmaf(ov.w, e, y.w);
		}
		const float inv = 1.0f / L;
		y.x *= inv;
		y.y *= inv;
		y.z *= inv;
		y.w *= inv;
		mx = fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w)));
	}
	const int e = ps_block_exponent(mx, bred);
	if (tid < items) ps_quantise(y, ps_pow2(23 - e), xd, items, tid);
	if (tid == 0) *s_xscale = ps_pow2(e - 23);
	__syncthreads();
}

// Phase E prologue: this CTA's rows of the activation vector (nq quads from act), polled until
// complete, quantised into xd (stride nq). nq <= 5 * PS_THREADS.
__device__ __noinline__ void ps_act_quant(const PsW w, int where, const float *act, int nq, uint32_t *xd, float *bred, float *s_xscale) {
	const int tid = threadIdx.x;
	__builtin_assume(__isShared(xd));
	__builtin_assume(__isShared(bred));
	__builtin_assume(__isShared(s_xscale));
	float4 v[5];
	int spins = 0;
	long long t0 = 0;
	bool ok;
	do {
		ok = true;
#pragma unroll
		for (int q = 0; q < 5; q++) {
			const int i = q * PS_THREADS + tid;
			v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
			if (i < nq) v[q] = ps_ld4(act + 4 * i);
			ok = ok && ps_ok(v[q]);
		}
	} while (!ok && ps_retry(w, where, spins, t0));
	float mx = 0.0f;
#pragma unroll
	for (int q = 0; q < 5; q++) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[q].x), fabsf(v[q].y)), fmaxf(fabsf(v[q].z), fabsf(v[q].w))));
	const int e = ps_block_exponent(mx, bred + PS_NW);
	const float qs = ps_pow2(23 - e);
#pragma unroll
	for (int q = 0; q < 5; q++) {
		const int i = q * PS_THREADS + tid;
		if (i < nq) ps_quantise(v[q], qs, xd, nq, i);
	}
	if (tid == 0) *s_xscale = ps_pow2(e - 23);
	__syncthreads();
}

// Phase B of one attention CTA = (head hh, cache slots j0 .. j1): q|k|v of this token from the hand-off
// vector (polled), q/k norm + RoPE, append of the new row (head 0's CTA of the chunk that holds `slot`),
// running-max softmax over the chunk (warp -> slots j0 + warp, + 12, ...; lane owns dims 4 lane.. and
// 128 + 4 lane..), merge of the 12 warps, (o[256], m, l) published to prow. att: 16 KB of scratch,
// wml: 3 * PS_NW floats. Reference: ops.hpp:224-370 (attention_decode), decode.hpp:203-211 (RoPE).
__device__ __noinline__ void ps_attention(const PsW w, int where, float *kcache, float *vcache, const float *rmsq, const float *rmsk,
                                          const float *cosr, const float *sinr, const float *qkv_ll, int QD, int hh, float *prow, int j0,
                                          int j1, int slot, float *att, float *wml, uint64_t keep) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	__builtin_assume(__isShared(att));
	__builtin_assume(__isShared(wml));
	float *wo = att, *qraw = att + PS_NW * AT_HD, *qs = qraw + 3 * AT_HD;
	float *wm = wml, *wl = wml + PS_NW, *we = wml + 2 * PS_NW;
	PsRope rr;
	if (warp < 2) ps_load_rope(rr, warp == 0 ? rmsq : rmsk, cosr, sinr, keep);
	// The cache rows do not depend on this token's q|k|v: a warp's first two rows are requested before
	// the poll (the new token's own row comes from shared memory later).
	float4 kv[2][4];
	auto load_keys = [&](int jb) {
#pragma unroll
		for (int u = 0; u < 2; u++) {
			const int j = jb + PS_NW * u;
			if (j < j1 && j != slot) {
				const float *kr = kcache + size_t(j) * AT_HD, *vr = vcache + size_t(j) * AT_HD;
				kv[u][0] = __ldcg(reinterpret_cast<const float4 *>(kr + 4 * lane));
				kv[u][1] = __ldcg(reinterpret_cast<const float4 *>(kr + 128 + 4 * lane));
				kv[u][2] = __ldcg(reinterpret_cast<const float4 *>(vr + 4 * lane));
				kv[u][3] = __ldcg(reinterpret_cast<const float4 *>(vr + 128 + 4 * lane));
			}
		}
	};
	load_keys(j0 + warp);
	if (tid < 3 * (AT_HD / 4)) {
		const float *src = qkv_ll + (tid < AT_HD / 4 ? hh * AT_HD + 4 * tid : QD + 4 * (tid - AT_HD / 4));
		float4 v;
		int spins = 0;
		long long t0 = 0;
		do {
			v = ps_ld4(src);
		} while (!ps_ok(v) && ps_retry(w, where, spins, t0));
		*reinterpret_cast<float4 *>(qraw + 4 * tid) = v;
	}
	__syncthreads();
	float *ks = qraw + AT_HD, *vs = qraw + 2 * AT_HD;
	// the reference scales q by 1/sqrt(256) before the dot products (ops.hpp:262,283); k is normed in place
	if (warp < 2) ps_norm_rope(qraw + warp * AT_HD, rr, warp == 0 ? 0.0625f : 1.0f, warp == 0 ? qs : ks);
	__syncthreads();
	if (hh == 0 && slot >= j0 && slot < j1 && tid < 2 * (AT_HD / 4)) {
		float *dst = (tid < AT_HD / 4 ? kcache : vcache) + size_t(slot) * AT_HD;
		const int j = tid & (AT_HD / 4 - 1);
		*reinterpret_cast<float4 *>(dst + 4 * j) = *reinterpret_cast<const float4 *>((tid < AT_HD / 4 ? ks : vs) + 4 * j);
	}
	const float4 q0 = *reinterpret_cast<const float4 *>(qs + 4 * lane);
	const float4 q1 = *reinterpret_cast<const float4 *>(qs + 128 + 4 * lane);
	float4 o0 = make_float4(0.f, 0.f, 0.f, 0.f), o1 = make_float4(0.f, 0.f, 0.f, 0.f);
	float m = -INFINITY, lsum = 0.0f;
#pragma unroll 1
	for (int jb = j0 + warp; jb < j1; jb += 2 * PS_NW) {
#pragma unroll
		for (int u = 0; u < 2; u++) {
			const int j = jb + PS_NW * u;
			if (j >= j1) continue;
			if (j == slot) {  // the new row: not in the cache yet for the other heads' CTAs
				kv[u][0] = *reinterpret_cast<const float4 *>(ks + 4 * lane);
				kv[u][1] = *reinterpret_cast<const float4 *>(ks + 128 + 4 * lane);
				kv[u][2] = *reinterpret_cast<const float4 *>(vs + 4 * lane);
				kv[u][3] = *reinterpret_cast<const float4 *>(vs + 128 + 4 * lane);
			}
			float t = q0.x * kv[u][0].x;
			t = fmaf(q0.y, kv[u][0].y, t);
			t = fmaf(q0.z, kv[u][0].z, t);
			t = fmaf(q0.w, kv[u][0].w, t);
			t = fmaf(q1.x, kv[u][1].x, t);
			t = fmaf(q1.y, kv[u][1].y, t);
			t = fmaf(q1.z, kv[u][1].z, t);
			t = fmaf(q1.w, kv[u][1].w, t);
			t = warp_sum(t);
			const float mn = fmaxf(m, t);
			const float corr = expf(m - mn);
			const float pp = expf(t - mn);
			lsum = fmaf(lsum, corr, pp);
			o0.x = fmaf(pp, kv[u][2].x, o0.x * corr);
			o0.y = fmaf(pp, kv[u][2].y, o0.y * corr);
			o0.z = fmaf(pp, kv[u][2].z, o0.z * corr);
			o0.w = fmaf(pp, kv[u][2].w, o0.w * corr);
			o1.x = fmaf(pp, kv[u][3].x, o1.x * corr);
			o1.y = fmaf(pp, kv[u][3].y, o1.y * corr);
			o1.z = fmaf(pp, kv[u][3].z, o1.z * corr);
			o1.w = fmaf(pp, kv[u][3].w, o1.w * corr);
			m = mn;
		}
		load_keys(jb + 2 * PS_NW);
	}
	if (lane == 0) {
		wm[warp] = m;
		wl[warp] = lsum;
	}
	*reinterpret_cast<float4 *>(wo + warp * AT_HD + 4 * lane) = o0;
	*reinterpret_cast<float4 *>(wo + warp * AT_HD + 128 + 4 * lane) = o1;
	__syncthreads();
	float M = -INFINITY;
#pragma unroll
	for (int i = 0; i < PS_NW; i++) M = fmaxf(M, wm[i]);
	if (tid < PS_NW) we[tid] = (wm[tid] == -INFINITY) ? 0.0f : expf(wm[tid] - M);
	__syncthreads();
	if (tid < AT_HD) {
		float O = 0.0f;
#pragma unroll
		for (int i = 0; i < PS_NW; i++) O = fmaf(wo[i * AT_HD + tid], we[i], O);
		ps_st(prow + tid, O);
	} else if (tid == AT_HD) {
		float Ls = 0.0f;
#pragma unroll
		for (int i = 0; i < PS_NW; i++) Ls = fmaf(wl[i], we[i], Ls);
		ps_st(prow + AT_HD, M);
		ps_st(prow + AT_HD + 1, Ls);
	}
	__syncthreads();  // the scratch is reused by phase C
}

// lm_head of one token: logits[v] = lm_scale[v] * sum_k x[k] W[k,v]; this CTA takes column tiles cta, cta + G, ...;
// a tile arrives as lm_nchunk ring stages in `ring`; warp w owns column groups 2w and 2w + 1 of every tile over
// all of its rows. Returns this lane's best (temperature-scaled) logit and the ring's barrier parities.
// pre: ring stages the caller has already requested (those that lie inside the up/gate region, which is
// idle from the last layer's up/gate product on).
struct PsLmOut {
	float best;
	int best_i;
	uint32_t plm, pemp;
};
__device__ __noinline__ PsLmOut ps_lm_head(const PsArgs &a, const PsW pw, uint8_t *ring, const uint32_t *xd, float xs, uint64_t *bar_lm,
                                           uint64_t *emp_lm, uint32_t plm, uint32_t pemp, uint64_t pol, uint64_t keep, int pre) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x, D = a.D, L = a.L;
	__builtin_assume(__isShared(ring));
	__builtin_assume(__isShared(xd));
	__builtin_assume(__isShared(bar_lm));
	__builtin_assume(__isShared(emp_lm));
float best = -INFINITY;  // running max of this lane's (temperature-scaled) logits, lanes 0..7
int best_i = -1;
{
	const int nst = a.lm_stages, nchunk = a.lm_nchunk, cq = a.lm_cq;
	const int my_tiles = (a.lm_ntiles - cta + G - 1) / G;
	const int total = my_tiles * nchunk;
	const uint32_t sbytes = uint32_t(a.lm_stage_bytes);
			auto issue_stage = [&](int q, int stg) {  // one lane
		const int t = cta + (q / nchunk) * G, c = q % nchunk;
		ps_issue(ring + size_t(stg) * sbytes, a.lm_tiled + (size_t(t) * nchunk + c) * sbytes, sbytes, &bar_lm[stg], pol, pw.s_abort);
	};
	if (tid == PS_THREADS - 32) {
#pragma unroll 1
		for (int s = pre; s < nst && s < total; s++) issue_stage(s, s);  // (the first `pre` stages were requested during the last layer)
	}
	PsAcc a0, a1;
	float sc = 0.0f;
	int stg = 0, c = 0, tile = cta;
	bool lm_rdy = false;
	const bool wact = 2 * warp < a.lm_groups;
#pragma unroll 1
	for (int q = 0; q < total; q++) {
		if (c == 0) {
#pragma unroll
			for (int i = 0; i < 12; i++) a0.v[i] = a1.v[i] = 0;
			const int v0 = tile * a.lm_groups * 4 + 8 * warp + lane;  // lanes 0..3: group 2w, lanes 4..7: group 2w+1
			sc = (wact && lane < 8 && v0 < a.V) ? ps_ldk(a.lm_scale + v0, keep) : 0.0f;
		}
		if (!lm_rdy) ps_wait_bulk(pw, (L << 4) | 6, &bar_lm[stg], (plm >> stg) & 1u);
		plm ^= (1u << stg);
		{  // the next stage's barrier is tested now; its result is needed only after this stage's products
			const int ns = (stg + 1 == nst) ? 0 : stg + 1;
			lm_rdy = (q + 1 < total) && ps_mbar_test(&bar_lm[ns], (plm >> ns) & 1u);
		}
		if (wact) {
			const uint4 *t0 = reinterpret_cast<const uint4 *>(ring + size_t(stg) * sbytes) + 2 * warp * cq;
			const uint32_t *x = xd + c * cq;
#pragma unroll 1
			for (int qq = lane; qq < cq; qq += 32) {
				const uint32_t x0 = x[qq], x1 = x[D / 4 + qq], x2 = x[2 * (D / 4) + qq];
				ps_mac(a0, t0[qq], x0, x1, x2);
				ps_mac(a1, t0[cq + qq], x0, x1, x2);
			}
		}
		__syncwarp();
		if (lane == 0) ps_mbar_arrive(&emp_lm[stg]);
		if (tid == PS_THREADS - 32) {
			const int nq = q + nst;
			if (nq < total) {
				ps_wait_bulk(pw, (L << 4) | 6, &emp_lm[stg], (pemp >> stg) & 1u);  // all 12 warps have left the stage
				issue_stage(nq, stg);
			}
		}
		__syncwarp();
		pemp ^= (1u << stg);
		if (c == nchunk - 1 && wact) {
			const float2 r01 = ps_finish2(a0, a1);  // lanes 0..3
			const float r1s = __shfl_sync(0xffffffffu, r01.y, lane & 3);  // every lane takes part in the shuffle
			const float r = (lane < 4) ? r01.x : r1s;
			const int v = tile * a.lm_groups * 4 + 8 * warp + lane;
			if (lane < 8 && v < a.V) {
				const float lg = (r * xs) * sc;
				__stcg(a.logits + v, lg);
				const float z = (a.sampler == 2) ? lg / a.temp : lg;
				if (z > best) {  // tiles ascend, so the first maximum keeps the lowest index
					best = z;
					best_i = v;
				}
			}
		}
		if (++stg == nst) stg = 0;
		if (++c == nchunk) {
			c = 0;
			tile += G;
		}
	}
}
	return PsLmOut{best, best_i, plm, pemp};
}

// Sampler of one token (0: none, 1: argmax, 2: min-p) over the logits row; `best`, `best_i` are this lane's
// candidates from the lm_head. Returns the sampled token (every thread) and the grid-barrier count.
struct PsSampOut {
	int tok;
	unsigned epoch;
};
__device__ __noinline__ PsSampOut ps_sampler(const PsArgs &a, const PsW pw, float best, int best_i, unsigned epoch, int n_logged, float *wm,
                                             int *s_cdf, float *s_f, int *s_i, float *bred, float *cbuf) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x, L = a.L;
	// these are shared-memory pointers: tell the compiler, or every access through them is a generic load
	__builtin_assume(__isShared(wm));
	__builtin_assume(__isShared(s_cdf));
	__builtin_assume(__isShared(s_f));
	__builtin_assume(__isShared(s_i));
	__builtin_assume(__isShared(bred));
	__builtin_assume(__isShared(cbuf));
const int wh = (L << 4) | 7;
int next_tok = 0;
if (a.sampler == 0) {
	ps_grid_sync(pw, wh, a.bar, a.bar_base + ++epoch * G);  // logits complete
} else {
	// CTA-local (max, argmax): value descending, index ascending; index -1 never beats a real one
	auto better = [](float v1, int i1, float v2, int i2) {
		if (v1 > v2) return true;
		if (v1 < v2) return false;
		if (i2 < 0) return i1 >= 0;
		if (i1 < 0) return false;
		return i1 < i2;
	};
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) {
		float ov = __shfl_xor_sync(0xffffffffu, best, o);
		int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
		if (better(ov, oi, best, best_i)) {
			best = ov;
			best_i = oi;
		}
	}
	if (lane == 0) {
		wm[warp] = best;
		s_cdf[warp] = best_i;
	}
	__syncthreads();
	if (tid == 0) {
		for (int i = 1; i < PS_NW; i++)
			if (better(wm[i], s_cdf[i], best, best_i)) {
				best = wm[i];
				best_i = s_cdf[i];
			}
		__stcg(a.samp_f + cta, best);
		__stcg(a.samp_i + cta, best_i);
	}
	ps_grid_sync(pw, wh, a.bar, a.bar_base + ++epoch * G);
	// every CTA reduces the per-CTA results the same way (warp 0)
	if (warp == 0) {
		float gmax = -INFINITY;
		int gidx = -1;
#pragma unroll 1
		for (int c = lane; c < G; c += 32) {
			float v = __ldcg(a.samp_f + c);
			int ix = __ldcg(a.samp_i + c);
			if (better(v, ix, gmax, gidx)) {
				gmax = v;
				gidx = ix;
			}
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) {
			float ov = __shfl_xor_sync(0xffffffffu, gmax, o);
			int oi = __shfl_xor_sync(0xffffffffu, gidx, o);
			if (better(ov, oi, gmax, gidx)) {
				gmax = ov;
				gidx = oi;
			}
		}
		if (lane == 0) {
			s_f[4] = gmax;
			s_i[0] = gidx;
		}
	}
	__syncthreads();
	const float gmax = s_f[4];
	const int gidx = s_i[0];
	if (a.sampler == 1) {
		next_tok = gidx;  // ops::argmax_logits (reference ops.hpp:744-760)
	} else {
		// ops::minp_logits (reference ops.hpp:762-859). z = logit / temp; rowmax = gmax;
		// p = exp(z - rowmax); maxp = exp(0) = 1 so cut = minp * 1; denom = sum of p >= cut.
		const float cut = a.minp * expf(gmax - gmax);
		float ds = 0.0f;
		{
			const int ntile = a.V / PS_SAMP_TILE;
			const int my_tiles = (ntile - cta + G - 1) / G;
#pragma unroll 1
			for (int j = tid; j < my_tiles * PS_SAMP_TILE; j += PS_THREADS) {
				const int v = (cta + (j / PS_SAMP_TILE) * G) * PS_SAMP_TILE + (j % PS_SAMP_TILE);
				const float pv = expf(__ldcg(a.logits + v) / a.temp - gmax);
				__stcg(a.probs + v, pv);
				ds += (pv < cut) ? 0.0f : pv;
			}
		}
		ds = block_sum<PS_NW>(ds, bred);
		if (tid == 0) __stcg(a.samp_f + G + cta, ds);
		ps_grid_sync(pw, wh, a.bar, a.bar_base + ++epoch * G);
		if (cta == 0) {
			// denominator: per-CTA sums added in a fixed tree by warp 0
			if (warp == 0) {
				float dv = 0.0f;
#pragma unroll 1
				for (int c = lane; c < G; c += 32) dv += __ldcg(a.samp_f + G + c);
				dv = warp_sum(dv);
				if (lane == 0) s_f[6] = 1.0f / dv;
			}
			float randf = 0.0f;
			const int rc = __ldcg(a.randf_count);
			if (rc < a.randf_cap) randf = __ldg(a.randf + rc);
			__syncthreads();
			const float inv = s_f[6];
			// inverse CDF: the first index whose sequential fp32 running sum reaches randf,
			// evaluated exactly and in parallel (cdf_cross_block) over chunks of probabilities
			// p = exp(z - max) * inv staged in the idle weight ring
			const int CH = a.samp_ch;
			if (tid == 0) {
				s_i[1] = -1;
				s_f[5] = 0.0f;
			}
			__syncthreads();
#pragma unroll 1
			for (int c0 = 0; c0 < a.V; c0 += CH) {
				const int n = min(CH, a.V - c0);
#pragma unroll 4
				for (int i = tid * 4; i < n; i += PS_THREADS * 4) {
					float4 v = __ldcg(reinterpret_cast<const float4 *>(a.probs + c0 + i));
					v.x *= inv;
					v.y *= inv;
					v.z *= inv;
					v.w *= inv;
					*reinterpret_cast<float4 *>(cbuf + i) = v;
				}
				__syncthreads();
				const int r = cdf_cross_block<PS_NW>(cbuf, n, &s_f[5], randf, s_cdf, c0 == 0 ? 1024 : 0);
				if (r >= 0) {
					if (tid == 0) s_i[1] = c0 + r;
					break;
				}
			}
			__syncthreads();
			if (tid == 0) {
				__stcg(a.samp_i + G, s_i[1] < 0 ? 0 : s_i[1]);
				*a.randf_count = rc + 1;
			}
		}
		ps_grid_sync(pw, wh, a.bar, a.bar_base + ++epoch * G);
		next_tok = __ldcg(a.samp_i + G);
	}
	if (cta == 0 && tid == 0) {
		if (a.tok_log && n_logged < a.log_cap) a.tok_log[n_logged] = next_tok;
		*a.tok = next_tok;
	}
	n_logged++;
}
	return PsSampOut{next_tok, epoch};
}

// Instrumentation of the DBG instantiation only: SM-clock stamps of one CTA along the last token,
// and progress marks of every warp in mapped host memory (for diagnosing a stall).
#define PS_BEACON(x)                                                                               \
	do {                                                                                           \
		if constexpr (DBG) {                                                                       \
			if (a.beacon && lane == 0) *(volatile int *)(a.beacon + cta * 16 + warp) = (lc << 8) | (x); \
		}                                                                                          \
	} while (0)
#define PS_GT(k)                                                                                        \
	do {                                                                                                \
		if constexpr (DBG) {                                                                            \
			if (a.gt && tid == 0 && !more && l == L / 2) {                                              \
				unsigned long long t_;                                                                  \
				asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
				a.gt[cta * 12 + (k)] = (long long)t_;                                                   \
			}                                                                                           \
		}                                                                                               \
	} while (0)
#define PS_GT_WARP(k)                                                                                   \
	do {                                                                                                \
		if constexpr (DBG) {                                                                            \
			if (a.gt && lane == 0 && !more && l == L / 2) {                                             \
				unsigned long long t_;                                                                  \
				asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
				a.gt[cta * 12 + (k)] = (long long)t_;                                                   \
			}                                                                                           \
		}                                                                                               \
	} while (0)
#define PS_STAMP()                                                       \
	do {                                                                 \
		if constexpr (DBG) {                                             \
			if (dbg_on && dbg_n < a.dbg_cap) a.dbg[dbg_n++] = clock64(); \
		}                                                                \
	} while (0)

template <bool DBG>
__global__ void __launch_bounds__(PS_THREADS, 1) decode_persist_kernel(const __grid_constant__ PsArgs a) {
	extern __shared__ uint8_t smem_raw[];
	uint8_t *smem = reinterpret_cast<uint8_t *>((uintptr_t(smem_raw) + 127) & ~uintptr_t(127));  // the host adds 128 bytes of slack
	__shared__ uint64_t bar_A, bar_C, bar_D, bar_E, bar_lm[8], emp_lm[8];
	__shared__ float bred[3 * PS_NW];
	__shared__ float s_part[PS_NW * 16];
	__shared__ int s_cnt[PS_NW + 4];
	__shared__ float s_xscale;
	__shared__ int s_abort;
	__shared__ float s_f[8];
	__shared__ int s_i[4];
	__shared__ int s_cdf[2 * PS_NW + 8];
	__shared__ float wm[3 * PS_NW];  // per-warp (m, l, weight) of the attention merge; also the sampler's per-warp maxima
	__shared__ PsLayer s_ly[PS_MAX_LAYERS];

#define R_A (smem + a.off_A)
#define R_C (smem + a.off_C)
#define R_D (smem + a.off_D)
#define R_E (smem + a.off_E)
	// (recomputed where they are used: a value that lives across the whole token loop costs a register, and the
	// registers this kernel cannot have are spilled to local memory, which the small L1 left beside 224 KB of
	// shared memory does not hold)
#define h (reinterpret_cast<float *>(smem + a.off_h))
#define xd (reinterpret_cast<uint32_t *>(smem + a.off_xd))
#define att (reinterpret_cast<float *>(smem + a.off_att))  /* wo[12][256] | qraw[768] (q_h, k, v) | qs[256] */
#define xd_s (ps_smem(smem + a.off_xd))
#define part_s (ps_smem(s_part))
#define cnt_s (ps_smem(s_cnt))
#define pol (ps_evict_first())
#define keep (ps_evict_last())

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x;
	const int D = a.D, L = a.L;

	if (tid == 0) {
		ps_mbar_init(&bar_A, 1);
		ps_mbar_init(&bar_C, 1);
		ps_mbar_init(&bar_D, 1);
		ps_mbar_init(&bar_E, 1);
#pragma unroll 1
		for (int i = 0; i < 8; i++) {
			ps_mbar_init(&bar_lm[i], 1);
			ps_mbar_init(&emp_lm[i], PS_NW);
		}
		s_abort = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (tid < PS_NW + 4) s_cnt[tid] = 0;
	{
		const int *src = reinterpret_cast<const int *>(a.layers);
		int *dst = reinterpret_cast<int *>(s_ly);
#pragma unroll 1
		for (int i = tid; i < L * int(sizeof(PsLayer) / 4); i += PS_THREADS) dst[i] = src[i];
	}
	__syncthreads();
	const PsW pw{&s_abort, a.err, a.wait_clocks, unsigned(a.poll_ns)};
	unsigned epoch = 0;  // grid barriers passed
	uint32_t pA = 0, pC = 0, pD = 0, pE = 0, plm = 0, pemp = 0;

	__shared__ PsCta s_c;
	{
		const int uA = cta - a.A.cta0, uC = cta - a.C.cta0, uD = cta - a.Dp.cta0, uE = cta - a.E.cta0;
		const bool hA = uA >= 0 && uA < a.A.units, hC = uC >= 0 && uC < a.C.units, hD = uD >= 0 && uD < a.Dp.units, hE = uE >= 0 && uE < a.E.units;
		if (tid == 0) {
			s_c.tileA = hA ? uA % a.A.ntiles : 0;
			s_c.tileC = hC ? uC % a.C.ntiles : 0;
			s_c.splitC = hC ? uC / a.C.ntiles : 0;
			s_c.tileE = hE ? uE % a.E.ntiles : 0;
			s_c.splitE = hE ? uE / a.E.ntiles : 0;
			s_c.presE = uE < 0 ? cta : cta - a.E.units;  // index of this CTA's presence word (if !hasE)
			s_c.uD = uD;
			// the unit this CTA fetches for a phase of layer l (one lane issues the copy)
			s_c.srcA = a.tiled + a.tl_A + size_t(hA ? uA : 0) * a.A.bytes;
			s_c.srcC = a.tiled + a.tl_C + size_t(hC ? uC : 0) * a.C.bytes;
			s_c.srcD = a.tiled + a.tl_D + size_t(hD ? uD : 0) * a.Dp.bytes;
			s_c.srcE = a.tiled + a.tl_E + size_t(hE ? uE : 0) * a.E.bytes;
			s_c.has = (hA ? 1 : 0) | (hC ? 2 : 0) | (hD ? 4 : 0) | (hE ? 8 : 0);
		}
		__syncthreads();
	}
#define hasA ((s_c.has & 1) != 0)
#define hasC ((s_c.has & 2) != 0)
#define hasD ((s_c.has & 4) != 0)
#define hasE ((s_c.has & 8) != 0)
#define tileA (s_c.tileA)
#define tileC (s_c.tileC)
#define splitC (s_c.splitC)
#define tileE (s_c.tileE)
#define splitE (s_c.splitE)
#define presE (s_c.presE)
#define uD (s_c.uD)
#define srcA (s_c.srcA)
#define srcC (s_c.srcC)
#define srcD (s_c.srcD)
#define srcE (s_c.srcE)

	if (tid == 0) {
		if (hasA) ps_issue(R_A, srcA, a.A.bytes, &bar_A, pol, &s_abort);
		if (hasC) ps_issue(R_C, srcC, a.C.bytes, &bar_C, pol, &s_abort);
		if (hasD && a.sched == 0) ps_issue(R_D, srcD, a.Dp.bytes, &bar_D, pol, &s_abort);
		if (hasE && a.sched == 0) ps_issue(R_E, srcE, a.E.bytes, &bar_E, pol, &s_abort);
	}

	int tok = __ldcg(a.tok);
	int pos = __ldcg(a.next_pos);
	const int rbase = __ldcg(a.ring_base);
	int n_logged = 0;
	int dbg_n = 0;
	// this lane's column in a product: group = warp / kp, column 4 * group + lane (lanes 0..3); active = the warp has a group
	const bool actA = hasA && warp / a.A.kp < a.A.ngroups, actC = hasC && warp / a.C.kp < a.C.ngroups;
	const bool actD = hasD && warp / a.Dp.kp < a.Dp.ngroups, actE = hasE && warp / a.E.kp < a.E.ngroups;
	const int colA = tileA * a.A.ngroups * 4 + (warp / a.A.kp) * 4 + (lane & 3);
	const int colC = tileC * a.C.ngroups * 4 + (warp / a.C.kp) * 4 + (lane & 3);
	const int colD = uD * a.Dp.ngroups * 4 + (warp / a.Dp.kp) * 4 + (lane & 3);
	const int colE = tileE * a.E.ngroups * 4 + (warp / a.E.kp) * 4 + (lane & 3);

	// ring stages of the lm_head that fit the up/gate region and belong to this CTA's first tile (chunks 0 .. lm_pre - 1)
	const int lm_pre = (cta < a.lm_ntiles && a.sched == 0) ? min(min(a.lm_stages, a.lm_nchunk), a.Dp.bytes / a.lm_stage_bytes) : 0;
#pragma unroll 1
	for (int step = 0; step < a.n_steps; step++) {
		const bool more = (step + 1 < a.n_steps);
		const bool dbg_on = DBG && (a.dbg != nullptr) && cta == a.dbg_cta && tid == 0 && !more;
		PS_STAMP();
		// ---------------------------------------------------------------- embedding
		if (a.force_ids) tok = __ldg(a.force_ids + step);
		if (tok < 0 || tok >= a.V) {
			if (tid == 0 && cta == 0) atomicExch(a.err, 1);
			tok = 0;
		}
#pragma unroll 1
		for (int d = tid; d < D; d += PS_THREADS) h[d] = a.wte_s[d] * (a.sqrtD * float(a.wte[size_t(tok) * D + d]));
		__syncthreads();

#pragma unroll 1
		for (int l = 0; l < L; l++) {
			const PsLayer &ly = s_ly[l];
			// position bookkeeping of this layer's cache (KVCache, reference decode.hpp:45-70)
			int p = pos, slot, valid;
			if (ly.is_local) {
				slot = (p - rbase) % ly.slots;
				valid = min(p + 1, ly.slots);
			} else {
				if (p >= ly.slots) {
					if (tid == 0 && cta == 0) atomicExch(a.err, 2);
					p = ly.slots - 1;
				}
				slot = p;
				valid = p + 1;
			}
			const int nch = ly.is_local ? a.nch_local : (valid <= 512 ? a.nch_local : (valid <= 2048 ? a.nch_mid : a.nch_long));
			const int nsA = AT_NH * nch;  // CTAs that take part in attention
			const int lc = step * L + l;
			const int nl = (l + 1 < L) ? l + 1 : (more ? 0 : -1);  // the layer whose units are fetched next
			float *const llb = a.ll + size_t(lc % 3) * a.ll_stride;
			float *const llprev = a.ll + size_t((lc + 2) % 3) * a.ll_stride;
			PS_BEACON(0x10);
			PS_GT(0);
			// ============================================================ A: QKV
			// Cold data of the whole layer (this lane's column scales, the norm weights of phase D) is requested
			// here, a phase or more before its use: a DRAM or L2 access issued while a burst of weight copies
			// lands can take microseconds, and a publishing warp that waits for its scale delays every consumer.
			float scA = 0.0f, scC = 0.0f, su_r = 0.0f, sg_r = 0.0f, scE = 0.0f;
			if (lane < 4) {
				if (actA) {
					const int n = colA;
					scA = ps_ldk(n < a.QD ? ly.sq + n : (n < a.QD + a.KD ? ly.sk + (n - a.QD) : ly.sv + (n - a.QD - a.KD)), keep);
				}
				if (actC) scC = ps_ldk(ly.so + colC, keep);
				if (actD) {
					su_r = ps_ldk(ly.su + colD, keep);
					sg_r = ps_ldk(ly.sg + colD, keep);
				}
				if (actE) scE = ps_ldk(ly.sd + colE, keep);
			}
			if (a.e_rows && hasE && lane < 4 * a.E.ngroups) scE = ps_ldk(ly.sd + tileE * a.E.ngroups * 4 + lane, keep);
			// The units were requested a layer ago: test their barriers early, so that the (long) latency of the
			// test hides behind the hand-off polls instead of following them.
			const bool rdyA = actA && ps_mbar_test(&bar_A, pA), rdyC = actC && ps_mbar_test(&bar_C, pC);
			{
				ps_resnorm(pw, (l << 4) | 1, D, h, xd, bred, &s_xscale, l > 0 ? llprev + a.ll_dn : nullptr, a.E.nsplit, llprev + a.ll_pres,
				           G - a.E.units, l > 0 ? s_ly[l - 1].mlp_post : nullptr, ly.attn_pre, keep, nullptr);
				PS_STAMP();
				PS_GT(1);
				PS_BEACON(0x11);
				if (actA) {
					if (!rdyA) ps_wait_bulk(pw, (l << 4) | 1, &bar_A, pA);
					PS_STAMP();
					const PsOut o = ps_product(ps_smem(R_A), a.A.ngroups, a.A.nq, a.A.kp, a.A.wq, false, xd_s, D / 4, part_s, cnt_s);
					if ((o.flags & 1) && lane < 4) ps_st(llb + a.ll_qkv + colA, (o.r0 * s_xscale) * scA);
					PS_STAMP();
					if ((o.flags & 2) && nl >= 0 && lane == 0) ps_issue(R_A, srcA + size_t(nl) * a.tl_layer, a.A.bytes, &bar_A, pol, &s_abort);
				} else {
					PS_STAMP();
					PS_STAMP();
				}
				pA ^= 1;
				if (a.sched == 1 && tid == 64) {  // (every warp passed the barrier that ended the prologue: the regions' last readers are long done)
					if (hasD) ps_issue(R_D, srcD + size_t(l) * a.tl_layer, a.Dp.bytes, &bar_D, pol, &s_abort);
					if (hasE) ps_issue(R_E, srcE + size_t(l) * a.tl_layer, a.E.bytes, &bar_E, pol, &s_abort);
				}
				PS_STAMP();
				PS_GT(2);
				PS_BEACON(0x12);
				// Wipe the arena copy of the NEXT layer. It was last used two layers ago; every CTA has
				// finished with it: this CTA got past the prologue above, which needs the down-projection
				// (or presence) words of ALL CTAs for the previous layer, and a CTA stores those after its
				// last read of anything older. The CTAs that idle through the attention phase wipe; the
				// fence orders the wipe before their own next down-projection / presence store.
				if (cta >= nsA) {
					float4 *other = reinterpret_cast<float4 *>(a.ll + size_t((lc + 1) % 3) * a.ll_stride);
					const int nw = G - nsA, n4 = a.ll_stride / 4, per = (n4 + nw - 1) / nw;
					const float e = __uint_as_float(PS_EMPTY);
#pragma unroll 1
					for (int i = (cta - nsA) * per + tid; i < min(n4, (cta - nsA + 1) * per); i += PS_THREADS)
						__stcg(other + i, make_float4(e, e, e, e));
					__syncthreads();
					if (tid == 0) __threadfence();
				}
				PS_STAMP();
			}
			// ============================================================ B: attention
			if (cta < nsA) {
				const int chunk = (valid + nch - 1) / nch;
				const int j0 = (cta >> 2) * chunk;
				ps_attention(pw, (l << 4) | 2, ly.kcache, ly.vcache, ly.rmsq, ly.rmsk, a.rope[ly.is_local][0] + size_t(p) * AT_HD,
				             a.rope[ly.is_local][1] + size_t(p) * AT_HD, llb + a.ll_qkv, a.QD, cta & 3,
				             llb + a.ll_att + (size_t(cta & 3) * PS_MAX_CH + (cta >> 2)) * PS_ATT_ROW, j0, min(valid, j0 + chunk), slot, att, wm,
				             keep);
			}
			PS_BEACON(0x24);
			PS_GT(3);
			PS_STAMP();
			// ============================================================ C: O projection
			{
				if (hasC) {
					const int hp = AT_NH / a.C.nsplit;
					ps_attn_merge(pw, (l << 4) | 3, llb + a.ll_att, splitC * hp, hp, nch, att, xd, bred, &s_xscale);
					PS_STAMP();
					PS_GT(4);
					PS_BEACON(0x31);
					if (actC && !rdyC) ps_wait_bulk(pw, (l << 4) | 3, &bar_C, pC);
					PS_STAMP();
					const PsOut o = ps_product(ps_smem(R_C), a.C.ngroups, a.C.nq, a.C.kp, a.C.wq, false, xd_s, hp * (AT_HD / 4), part_s, cnt_s);
					if ((o.flags & 1) && lane < 4) ps_st(llb + a.ll_op + size_t(splitC) * D + colC, (o.r0 * s_xscale) * scC);
					if (o.flags & 2) PS_GT_WARP(10);
					PS_STAMP();
					if ((o.flags & 2) && nl >= 0 && lane == 0) ps_issue(R_C, srcC + size_t(nl) * a.tl_layer, a.C.bytes, &bar_C, pol, &s_abort);
				} else {
					PS_STAMP();
					PS_STAMP();
					PS_STAMP();
				}
				pC ^= 1;
				PS_STAMP();
				PS_GT(5);
				PS_BEACON(0x32);
			}
			// ============================================================ D: up & gate + GeGLU
			{
				const bool rdyD = actD && ps_mbar_test(&bar_D, pD);
				ps_resnorm(pw, (l << 4) | 4, D, h, xd, bred, &s_xscale, llb + a.ll_op, a.C.nsplit, nullptr, 0, ly.attn_post, ly.mlp_pre, keep, nullptr,
				           (DBG && a.dbg && cta == a.dbg_cta && !more && l == L / 2) ? a.dbg + 3930 : nullptr);
				PS_STAMP();
				PS_GT(6);
				PS_BEACON(0x41);
				if (actD && !rdyD) ps_wait_bulk(pw, (l << 4) | 4, &bar_D, pD);
				PS_STAMP();
				if (hasD) {
					const PsOut o = ps_product(ps_smem(R_D), a.Dp.ngroups, a.Dp.nq, a.Dp.kp, a.Dp.wq, true, xd_s, D / 4, part_s, cnt_s);
					if ((o.flags & 1) && lane < 4) {
						const float xs = s_xscale;
						ps_st(llb + a.ll_act + colD, ps_gelu(a.lut, (o.r1 * xs) * sg_r, keep) * ((o.r0 * xs) * su_r));
					}
				}
				pD ^= 1;
				PS_STAMP();
				PS_GT(7);
				PS_BEACON(0x42);
			}
			// ============================================================ E: down projection
			{
				const bool rdyE = hasE && ps_mbar_test(&bar_E, pE);
				if (a.e_rows && hasE) {
					// no prologue: every warp polls and quantises its own rows inside the product
					PS_STAMP();
					PS_GT(8);
					PS_BEACON(0x51);
					if (!rdyE) ps_wait_bulk(pw, (l << 4) | 5, &bar_E, pE);
					PS_STAMP();
					const PsOut o = ps_product_rows(pw, (l << 4) | 5, ps_smem(R_E), a.E.ngroups, a.E.nq, a.e_wq, llb + a.ll_act + size_t(splitE) * a.E.nq * 4,
					                                part_s, cnt_s + 4u * (PS_NW + 2),
					                                (DBG && a.dbg && cta == a.dbg_cta && !more && l == L / 2) ? a.dbg + 3800 : nullptr);
					if ((o.flags & 1) && lane < 4 * a.E.ngroups && cta != a.fault_cta)
						ps_st(llb + a.ll_dn + size_t(splitE) * D + tileE * a.E.ngroups * 4 + lane, o.r0 * scE);
					if (o.flags & 2) PS_GT_WARP(11);
					PS_STAMP();
					// every warp has left the up/gate product and this one: both regions are free
					if (a.sched == 0 && (o.flags & 2) && l + 1 < L && lane == 0) {
						ps_issue(R_E, srcE + size_t(l + 1) * a.tl_layer, a.E.bytes, &bar_E, pol, &s_abort);
						if (hasD) ps_issue(R_D, srcD + size_t(l + 1) * a.tl_layer, a.Dp.bytes, &bar_D, pol, &s_abort);
					}
				} else {
				if (hasE) {
					ps_act_quant(pw, (l << 4) | 5, llb + a.ll_act + size_t(splitE) * a.E.nq * 4, a.E.nq, xd, bred, &s_xscale);
				} else {
					__syncthreads();  // every warp has left the up/gate product
				}
				// the up/gate region is free: request the next layer's unit now that the hand-off loads are done
				if (a.sched == 0 && tid == 32 && hasD && l + 1 < L) ps_issue(R_D, srcD + size_t(l + 1) * a.tl_layer, a.Dp.bytes, &bar_D, pol, &s_abort);
				if (tid == 32 && l + 1 == L) {
					// last layer: the up/gate region is idle until the lm_head, whose ring starts there. Its first stages
					// are requested now, so that they land under the down projection and the final norm.
#pragma unroll 1
					for (int sg = 0; sg < lm_pre; sg++)
						ps_issue(R_D + size_t(sg) * a.lm_stage_bytes, a.lm_tiled + (size_t(cta) * a.lm_nchunk + sg) * a.lm_stage_bytes, uint32_t(a.lm_stage_bytes),
						         &bar_lm[sg], pol, &s_abort);
				}
				PS_STAMP();
				PS_GT(8);
				PS_BEACON(0x51);
				if (hasE) {
					if (actE && !rdyE) ps_wait_bulk(pw, (l << 4) | 5, &bar_E, pE);
					PS_STAMP();
					const PsOut o = ps_product(ps_smem(R_E), a.E.ngroups, a.E.nq, a.E.kp, a.E.wq, false, xd_s, a.E.nq, part_s, cnt_s);
					if ((o.flags & 1) && lane < 4 && cta != a.fault_cta) ps_st(llb + a.ll_dn + size_t(splitE) * D + colE, (o.r0 * s_xscale) * scE);
					if (o.flags & 2) PS_GT_WARP(11);
					PS_STAMP();
					if (a.sched == 0 && (o.flags & 2) && l + 1 < L && lane == 0) ps_issue(R_E, srcE + size_t(l + 1) * a.tl_layer, a.E.bytes, &bar_E, pol, &s_abort);
				} else {
					if (tid == 0) ps_st(llb + a.ll_pres + presE, 0.0f);
					PS_STAMP();
					PS_STAMP();
				}
				}
				pE ^= 1;
				PS_STAMP();
				PS_GT(9);
				PS_BEACON(0x52);
			}
		}

		// ================================================================ lm_head
		// logits[v] = lm_scale[v] * sum_k x[k] W[k,v]; this CTA takes column tiles cta, cta + G, ...;
		// a tile arrives as lm_nchunk ring stages laid over the (now idle) up/gate and down regions;
		// warp w owns column groups 2w and 2w + 1 of every tile over all of its rows.
		const int lc = step * L + L;
		{
			float *const lllast = a.ll + size_t((lc + 2) % 3) * a.ll_stride;
			ps_resnorm(pw, (L << 4) | 6, D, h, xd, bred, &s_xscale, lllast + a.ll_dn, a.E.nsplit, lllast + a.ll_pres, G - a.E.units,
			           s_ly[L - 1].mlp_post, a.final_norm, keep, cta == 0 ? a.xnorm_out : nullptr);
		}
		PS_STAMP();
		PS_BEACON(0x61);
		const PsLmOut lo = ps_lm_head(a, pw, R_D, xd, s_xscale, bar_lm, emp_lm, plm, pemp, pol, keep, lm_pre);
		plm = lo.plm;
		pemp = lo.pemp;
		__syncthreads();

		// ================================================================ sampler
		PS_STAMP();
		PS_BEACON(0x70);
		const PsSampOut so = ps_sampler(a, pw, lo.best, lo.best_i, epoch, n_logged, wm, s_cdf, s_f, s_i, bred, reinterpret_cast<float *>(R_D));
		const int next_tok = so.tok;
		epoch = so.epoch;
		if (a.sampler != 0) n_logged++;
		PS_STAMP();
		PS_BEACON(0x7F);
		pos += 1;
		if (cta == 0 && tid == 0) *a.next_pos = pos;
		// the ring is idle again: fetch the next token's layer-0 up/gate and down units
		if (tid == 0 && more && a.sched == 0) {
			if (hasD) ps_issue(R_D, srcD, a.Dp.bytes, &bar_D, pol, &s_abort);
			if (hasE) ps_issue(R_E, srcE, a.E.bytes, &bar_E, pol, &s_abort);
		}
		tok = next_tok;
		if (__syncthreads_or(*(volatile int *)&s_abort)) break;  // the whole CTA leaves together
	}
	if (*(volatile int *)&s_abort) {
		// gave up: let the bulk copies still in flight land in this CTA's shared memory before it returns
		const long long t0 = clock64();
		while (clock64() - t0 < 400000) {
		}
		__syncthreads();
	}
	if (cta == 0 && tid == 0 && a.log_count) *a.log_count = n_logged;
	// Leave the hand-off arena as the next launch expects it: copy 0 empty (copies 1 and 2 are wiped during
	// its layers 0 and 1, like every copy a layer before its use). Every CTA is past the last token's grid
	// barriers, which all CTAs reach only after their last read of the arena.
	if (!*(volatile int *)&s_abort) {
		float4 *c0 = reinterpret_cast<float4 *>(a.ll);
		const int n4 = a.ll_stride / 4, per = (n4 + G - 1) / G;
		const float e = __uint_as_float(PS_EMPTY);
#pragma unroll 1
		for (int i = cta * per + tid; i < min(n4, (cta + 1) * per); i += PS_THREADS) __stcg(c0 + i, make_float4(e, e, e, e));
	}
#undef h
#undef xd
#undef att
#undef xd_s
#undef part_s
#undef cnt_s
#undef pol
#undef keep
#undef R_A
#undef R_C
#undef R_D
#undef R_E
#undef hasA
#undef hasC
#undef hasD
#undef hasE
#undef tileA
#undef tileC
#undef splitC
#undef tileE
#undef splitE
#undef presE
#undef uD
#undef srcA
#undef srcC
#undef srcD
#undef srcE
}

}  // namespace tg
