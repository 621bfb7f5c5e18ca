// Persistent decode kernel: the whole per-token forward (and the sampler) of
// one sequence in ONE cooperative launch, one CTA per SM.
//
// Why: at batch 1 a Gemma-3-1B layer is only 26.8 MB of int8 weights — 4 us of
// HBM time — split over five dependent phases. Separate kernels cost more in
// launch gaps and cold starts than the data movement itself. Here
//   * every CTA owns a fixed slice of each weight matrix (a column strip, or a
//     column strip x K-split), stored contiguously in a re-tiled copy of the
//     layer weights, and fetches it with bulk copies (cp.async.bulk) into a
//     shared-memory region reserved for that phase. A region is refilled for
//     the NEXT layer after the current layer has consumed it, so about one
//     layer of weights per SM (186 KB) is always in flight and HBM never waits
//     for the dependency chain;
//   * phases hand over through small L2-resident vectors that validate
//     themselves (a sentinel marks words not yet written), one grid barrier
//     per layer (one atomic counter, bounded spin);
//   * RMSNorms are recomputed redundantly by every CTA from those vectors, and
//     the residual stream lives in each CTA's shared memory;
//   * split-K partial sums are written once and summed in split order by their
//     consumers: no floating-point atomics, results are run-to-run identical.
//
// Phases per layer (reference modules.hpp:135-169, 203-220):
//   A  pre-norm + Q|K|V matvec            -> partial sums
//   B  q/k norm, RoPE, KV append, split-KV attention -> (m, l, o) partials
//   C  attention merge + O matvec         -> partial sums
//   D  post-norm + residual + pre-norm + up & gate matvec + LUT-GeGLU -> act
//   E  down matvec                        -> partial sums
// then the lm_head (final residual + norm in its prologue, logits streamed
// through a TMA ring) and the sampler (argmax, or min-p with the sequential
// fp32 inverse CDF of reference ops.hpp:848-858 evaluated by an exact scan).
//
// Every wait is bounded: a spin that runs out sets *err and a shared abort
// flag, after which all waits fall through and the kernel returns.
#pragma once
#include <cuda.h>

#include "kernels_decode.cuh"
#include "kernels_sampler.cuh"
#include "tg_common.cuh"

namespace tg {

constexpr int MG_THREADS = 384;
constexpr int MG_NWARPS = MG_THREADS / 32;
constexpr int MG_SPIN_CAP = 1 << 22;
constexpr int MG_LM_STAGES = 3;
constexpr int MG_LM_TN = 128;
constexpr int MG_MAX_ATT = 64;  // most CTAs that take part in attention

struct MgPhase {
	int TN;        // columns (bytes per row) of a tile, multiple of 16
	int segs;      // TN / 16
	int nsplit;    // K-splits
	int kc;        // rows per split
	int box_rows;  // rows per TMA box (<= 256, divides kc)
	int nboxes;    // kc / box_rows
	int ntiles;    // column tiles
	int units;     // ntiles * nsplit (<= grid size)
	int bytes;     // shared-memory bytes of this phase's region
	// thread mapping constants (integer division by a run-time value costs ~100 clk per use, and the tile
	// helpers need two or three of them per call): rstep = 384 / segs, m_x = ceil(2^32 / x) for __umulhi
	int rstep;
	unsigned m_segs, m_rstep;
};

struct MgLayer {
	const float *sq, *sk, *sv, *so, *su, *sg, *sd;  // per-column scales
	const float *rmsq, *rmsk, *attn_pre, *attn_post, *mlp_pre, *mlp_post;
	float *kcache, *vcache;
	int slots, is_local;
};
constexpr int MG_MAX_LAYERS = 32;

struct MgArgs {
	const CUtensorMap *tmaps;  // [0] = lm_head
	const int8_t *tiled;       // re-tiled layer weights: per layer [A units | C units | D units (up, gate) | E units]
	size_t tl_layer, tl_A, tl_C, tl_D, tl_E;  // layer stride and byte offsets of the phases inside a layer
	const MgLayer *layers;
	int L, D, I, V, QD, KD;
	MgPhase A, C, Dp, E, LM;
	int tm_lm;
	int lm_bps;  // TMA boxes per lm_head ring stage
	const float *lm_scale, *final_norm;
	const int8_t *wte;
	const float *wte_s;
	float sqrtD;
	const float *rope[2][2];  // [is_local][cos, sin]
	GeluLut lut;
	// shared-memory carve-up (byte offsets from a 1024-aligned base)
	int off_A, off_C, off_D, off_E, off_h, off_xs, off_red, off_att, smem_total;
	// L2-resident exchange buffers
	// Self-validating hand-off arena, two copies used by alternate layers: every float is
	// either the sentinel MG_LL_EMPTY or a value. ll + parity * ll_stride + one of the offsets:
	//   ll_pA  [A.nsplit][NQ]  K-split partial sums of q|k|v        (A -> B)
	//   ll_att [MG_MAX_ATT][4*256 + 8] attention partials (o, m, l) (B -> C)
	//   ll_pC  [C.nsplit][D]   K-split partial sums of the O projection (C -> D)
	//   ll_act [I]             GeGLU activations                    (D -> E)
	float *ll;
	int ll_stride, ll_pA, ll_att, ll_pC, ll_act;
	// Down projection -> next layer: {value, tag} words (8-byte stores are single-copy atomic), two
	// buffers alternating by layer, each [E.nsplit][D] words followed by one presence word for every
	// CTA that holds no down-projection unit. A word is valid when its tag is the layer's tag.
	uint2 *pe;
	int pe_stride;   // words per buffer
	unsigned seq0;   // layer tags of this launch start above seq0
	float *logits;                    // [V]
	float *probs;                     // [V] exp(z - max) of the min-p sampler (before normalisation)
	int samp_ch;                      // probabilities staged per round of the inverse CDF (multiple of 4, fits the weight ring)
	float *samp_f;                    // [3][grid] sampler partials
	int *samp_i;                      // [grid]
	float *xnorm_out;                 // [D] final-normed hidden state (parity read-back)
	unsigned *bar;                    // grid barrier counter, zero at launch
	int *err;
	int *tok;        // token to feed / last sampled
	int *next_pos;   // position of the next token
	int *ring_base;
	int *tok_log;    // [log_cap] sampled tokens
	int *log_count;
	int log_cap;
	int n_steps;
	int sampler;     // 0 none (logits only), 1 argmax, 2 min-p
	float minp, temp;
	const float *randf;
	int *randf_count;
	int randf_cap;
	int att_local, att_global;  // CTAs taking part in attention
	long long *dbg;  // optional: SM-clock stamps of one CTA along the last step (profiling aid)
	int dbg_cta;     // which CTA records
	int sched;       // when the next layer's large tiles are requested. Bit 0: up/gate after the down projection's poll (else
	                 // right after the gate product); bit 1: down tiles after phase A's prologue (else after the down
	                 // product). A burst of bulk copies delays whatever runs while it lands (hand-off loads by up to
	                 // ~1 us, tile products by ~0.3 us); other placements that were measured (paced pieces at ten points
	                 // of the layer, fetching during the attention phase, landing only under the tile products) moved
	                 // the cost around without lowering it.
	int dbg_cap;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok)
	    : "r"(smem_u32(bar)), "r"(parity)
	    : "memory");
	return ok != 0;
}
// 2-D tiled TMA load into this CTA only (never cluster-wide): box at (x = byte column, y = row) -> dst, completes on bar.
// Weights are read once per token, so they carry an L2 evict-first policy and
// leave the L2 to the KV cache and the small exchange vectors.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
	uint64_t pol;
	asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
	return pol;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar, uint64_t pol) {
	asm volatile(
	    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], "
	    "[%4], %5;" ::"r"(smem_u32(dst)),
	    "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
	    : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
	unsigned v;
	asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

// Self-validating hand-off ("LL" style): the consumer's buffer is filled with a sentinel that no
// computation produces (all ones, a NaN the hardware never generates); the producer stores plain
// values; the consumer loads the data itself and repeats a load until none of its words is the
// sentinel. 4-byte accesses are single-copy atomic, so a word is either old (sentinel) or new.
// One L2 round trip hands the data over; no flag, no fence, no counter.
__device__ __forceinline__ void st_tagged(uint2 *p, float v, unsigned tag) {
	asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2(const uint2 *p) {  // two consecutive {value, tag} words
	uint4 r;
	asm volatile("ld.relaxed.gpu.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
	return r;
}
__device__ __forceinline__ uint2 ld_tagged_acquire(const uint2 *p) {
	uint2 r;
	asm volatile("ld.acquire.gpu.global.v2.b32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
	return r;
}
constexpr unsigned MG_LL_EMPTY = 0xFFFFFFFFu;
__device__ __forceinline__ void ll_store(float *p, float v) {
	asm volatile("st.relaxed.gpu.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ float4 ll_load4_once(const float *p) {
	float4 r;
	asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p) : "memory");
	return r;
}
__device__ __forceinline__ bool ll_valid(const float4 &v) {
	return __float_as_uint(v.x) != MG_LL_EMPTY && __float_as_uint(v.y) != MG_LL_EMPTY &&
	       __float_as_uint(v.z) != MG_LL_EMPTY && __float_as_uint(v.w) != MG_LL_EMPTY;
}

struct MgCtx {
	int *s_abort;  // shared flag
	int *err;      // global flag
	unsigned *bar;
	unsigned epoch;  // barriers passed so far
	unsigned G;
};

// wait for a TMA region; every thread polls (the barrier word is in shared memory)
__device__ __forceinline__ void mg_wait_tma(MgCtx &c, uint64_t *bar, uint32_t parity) {
	if (*(volatile int *)c.s_abort) return;
	int spins = 0;
	while (!mbar_try_wait(bar, parity)) {
		if (++spins > MG_SPIN_CAP) {
			*c.s_abort = 1;
			atomicExch(c.err, 3);
			return;
		}
	}
}

// Polling discipline of the self-validating hand-off: a batch of loads is issued, and if any
// word is still empty the WHOLE batch is reloaded after a short pause (compact code; the retry is
// the rare path). ll_retry() counts the rounds and gives up after MG_SPIN_CAP of them.
__device__ __noinline__ bool ll_retry(MgCtx &c, int &spins) {
	if (*(volatile int *)c.s_abort) return false;
	if (++spins > MG_SPIN_CAP) {
		*c.s_abort = 1;
		atomicExch(c.err, 5);
		return false;
	}
	__nanosleep(20);
	return true;
}

// grid-wide barrier, split so that work which does not depend on other CTAs
// (TMA issue for the next layer, cold-vector prefetch) runs between the two
// halves: arrive (release) ... wait (acquire, bounded spin).
struct MgBar {
	unsigned old, target;
};
__device__ __forceinline__ void mg_arrive(MgCtx &c, MgBar &b) {
	__syncthreads();
	c.epoch += 1;
	b.target = c.epoch * c.G;
	b.old = 0;
	if (threadIdx.x == 0) {
		__threadfence();
		b.old = atomicAdd(c.bar, 1u);
	}
}
__device__ __noinline__ void mg_wait(MgCtx &c, const MgBar &b) {
	if (threadIdx.x == 0) {
		if (b.old + 1u < b.target && !*(volatile int *)c.s_abort) {  // the last arriver need not poll
			int spins = 0;
			while (ld_acquire_u32(c.bar) < b.target) {
				if (++spins > MG_SPIN_CAP) {
					*c.s_abort = 1;
					atomicExch(c.err, 4);
					break;
				}
			}
		}
	}
	__syncthreads();
}
__device__ __forceinline__ void mg_grid_sync(MgCtx &c) {
	MgBar b;
	mg_arrive(c, b);
	mg_wait(c, b);
}

template <int NW>
__device__ __forceinline__ float mg_block_sum(float v, float *red) {
	v = warp_sum(v);
	__syncthreads();
	if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
	__syncthreads();
	float t = 0.0f;
#pragma unroll
	for (int w = 0; w < NW; w++) t += red[w];
	return t;
}

// ------------------------------------------------------------------ tile arithmetic
// sm_100 packed fp32: two IEEE fp32 operations per instruction, same rounding as the scalar forms
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
	float2 d;
	asm("fma.rn.f32x2 %0, %1, %2, %3;"
	    : "=l"(*reinterpret_cast<uint64_t *>(&d))
	    : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)), "l"(*reinterpret_cast<uint64_t *>(&c)));
	return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
	float2 d;
	asm("add.rn.f32x2 %0, %1, %2;"
	    : "=l"(*reinterpret_cast<uint64_t *>(&d))
	    : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
	return d;
}

// acc[n] += x * float(int8 n) for the 16 int8 of v. The integer pipe (PRMT) runs
// at half the fp32 rate on this part, so the fp32 side is packed two-wide.
__device__ __forceinline__ void mg_fma16(float (&acc)[16], const int4 &v, float x) {
	const uint32_t words[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
	const float2 x2 = make_float2(x, x), c2 = make_float2(-8388736.0f, -8388736.0f);
#pragma unroll
	for (int j = 0; j < 4; j++) {
		const uint32_t b = words[j] ^ 0x80808080u;
		float2 f01 = make_float2(__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7650u)),
		                         __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7651u)));
		float2 f23 = make_float2(__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7652u)),
		                         __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7653u)));
		f01 = fadd2(f01, c2);
		f23 = fadd2(f23, c2);
		float2 a01 = make_float2(acc[4 * j], acc[4 * j + 1]), a23 = make_float2(acc[4 * j + 2], acc[4 * j + 3]);
		a01 = ffma2(x2, f01, a01);
		a23 = ffma2(x2, f23, a23);
		acc[4 * j] = a01.x;
		acc[4 * j + 1] = a01.y;
		acc[4 * j + 2] = a23.x;
		acc[4 * j + 3] = a23.y;
	}
}

// Tile [rows][TN bytes] densely packed in shared memory, TN = 16 * segs. A thread
// owns one 16-byte column group and every RG-th row (RG = 384 / segs):
//   segs a power of two: thread t -> group t % segs, first row t / segs. A warp
//     reads 32 consecutive 16-byte pieces (conflict-free) and holds all groups;
//   otherwise (48-byte rows): thread t -> group t / RG, first row t % RG, so a
//     warp holds ONE group; its lanes read rows 48 bytes apart, which is also
//     conflict-free because 48 is an odd multiple of 16.
// Either way piece (row, group) sits at 16 * (row * segs + group) and a thread
// advances by 16 * 384 bytes per step.
__device__ __forceinline__ bool mg_seg_major(int segs) { return (segs & (segs - 1)) != 0; }

__device__ __forceinline__ void mg_tile_dot(float (&acc)[16], const uint8_t *tile, int rows, const MgPhase &ph, const float *xs) {
	const int segs = ph.segs, rstep = ph.rstep;
	int row, grp;
	if (mg_seg_major(segs)) {
		grp = int(__umulhi(threadIdx.x, ph.m_rstep));
		row = threadIdx.x - grp * rstep;
	} else {
		row = segs == 1 ? int(threadIdx.x) : int(__umulhi(threadIdx.x, ph.m_segs));  // (2^32 / 1 does not fit the constant)
		grp = threadIdx.x - row * segs;
	}
	const uint8_t *p = tile + 16 * (row * segs + grp);
	const int pstep = 16 * MG_THREADS;
#pragma unroll 1
	for (; row + 3 * rstep < rows; row += 4 * rstep) {
		int4 v0 = *reinterpret_cast<const int4 *>(p);
		int4 v1 = *reinterpret_cast<const int4 *>(p + pstep);
		int4 v2 = *reinterpret_cast<const int4 *>(p + 2 * pstep);
		int4 v3 = *reinterpret_cast<const int4 *>(p + 3 * pstep);
		float x0 = xs[row], x1 = xs[row + rstep], x2 = xs[row + 2 * rstep], x3 = xs[row + 3 * rstep];
		p += 4 * pstep;
		mg_fma16(acc, v0, x0);
		mg_fma16(acc, v1, x1);
		mg_fma16(acc, v2, x2);
		mg_fma16(acc, v3, x3);
	}
#pragma unroll 1
	for (; row < rows; row += rstep) {
		int4 v0 = *reinterpret_cast<const int4 *>(p);
		p += pstep;
		mg_fma16(acc, v0, xs[row]);
	}
}

// Sum the per-thread column sums over all threads of the same column group.
// Inside a warp the 16 values are reduced by halving: in the round with lane
// distance `off` a lane keeps one half of its values and receives the partner's
// sums for that half, so the rounds cost 8 + 4 + 2 + 1 shuffles instead of 16
// each (the shuffle unit issues one warp instruction per clock per SM). The
// per-warp results meet in `red` ([12][TN] floats). Returns the total of column
// threadIdx.x for threads < TN. The order of additions is fixed.
__device__ __forceinline__ float mg_tile_reduce(float (&v)[16], const MgPhase &ph, float *red) {
	const int segs = ph.segs;
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const bool sm = mg_seg_major(segs);
	const int TN = 16 * segs;
	int base = 0, nv = 16;
	{
		const bool up = lane & 16;
#pragma unroll
		for (int i = 0; i < 8; i++) {
			const float send = up ? v[i] : v[i + 8];
			const float keep = up ? v[i + 8] : v[i];
			v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
		}
		base += up ? 8 : 0;
		nv = 8;
	}
	if (sm || segs <= 8) {
		const bool up = lane & 8;
#pragma unroll
		for (int i = 0; i < 4; i++) {
			const float send = up ? v[i] : v[i + 4];
			const float keep = up ? v[i + 4] : v[i];
			v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
		}
		base += up ? 4 : 0;
		nv = 4;
	}
	if (sm || segs <= 4) {
		const bool up = lane & 4;
#pragma unroll
		for (int i = 0; i < 2; i++) {
			const float send = up ? v[i] : v[i + 2];
			const float keep = up ? v[i + 2] : v[i];
			v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
		}
		base += up ? 2 : 0;
		nv = 2;
	}
	if (sm || segs <= 2) {
		const bool up = lane & 2;
		const float send = up ? v[0] : v[1];
		const float keep = up ? v[1] : v[0];
		v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
		base += up ? 1 : 0;
		nv = 1;
	}
	bool writer = true;
	if (sm || segs <= 1) {
		v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
		writer = (lane & 1) == 0;
	}
	const int grp = sm ? int(__umulhi(threadIdx.x, ph.m_rstep)) : (lane & (segs - 1));
	__syncthreads();  // `red` may still be read from a previous use
	if (writer) {
#pragma unroll
		for (int i = 0; i < 8; i++)
			if (i < nv) red[warp * TN + grp * 16 + base + i] = v[i];
	}
	__syncthreads();
	float s = 0.0f;
	if (int(threadIdx.x) < TN) {
		if (sm) {
			const int g = threadIdx.x >> 4, wpg = ph.rstep >> 5;  // column group, warps per group
			for (int w = g * wpg; w < (g + 1) * wpg; w++) s += red[w * TN + threadIdx.x];
		} else {
#pragma unroll
			for (int w = 0; w < MG_NWARPS; w++) s += red[w * TN + threadIdx.x];
		}
	}
	return s;
}

// One shared copy of "tile . x -> column sums": the phases run once per layer,
// so inlining this at every call site only thrashes the instruction cache.
__device__ __noinline__ float mg_tile_colsum(const uint8_t *tile, int rows, const MgPhase &ph, const float *xs, float *red) {
	float acc[16];
#pragma unroll
	for (int i = 0; i < 16; i++) acc[i] = 0.0f;
	mg_tile_dot(acc, tile, rows, ph, xs);
	return mg_tile_reduce(acc, ph, red);
}

// TMA issue for one phase region: `nmat` matrices (1, or 2 for up+gate), each
// nboxes boxes of box_rows rows at byte column x, rows from y0.
// Untiled bulk copy global -> this CTA's shared memory, completing on an mbarrier. Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
	asm volatile(
	    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
	    "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
	    : "memory");
}
// A CTA's unit of a weight matrix is one contiguous block of the re-tiled weight copy (see
// retile_kernel): the whole region is fetched with a few large sequential copies. Called by every
// lane of one warp: lane 0 arms the barrier, then lane i issues piece i.
constexpr uint32_t MG_BULK_PIECE = 16384;
__device__ __noinline__ void mg_issue(uint8_t *dst, const int8_t *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
	const int lane = threadIdx.x & 31;
	if (lane == 0) {
		fence_proxy_async();
		mbar_expect_tx(bar, bytes);
	}
	__syncwarp();
	for (uint32_t off = lane * MG_BULK_PIECE; off < bytes; off += 32 * MG_BULK_PIECE)
		bulk_load(dst + off, src + off, min(MG_BULK_PIECE, bytes - off), bar, pol);
}
__device__ __forceinline__ void mg_issue_A(const MgArgs &a, const MgLayer *, int l, int cta, uint8_t *dst, uint64_t *bar,
                                           uint64_t pol) {
	if (cta >= a.A.units) return;
	mg_issue(dst, a.tiled + size_t(l) * a.tl_layer + a.tl_A + size_t(cta) * a.A.bytes, a.A.bytes, bar, pol);
}
__device__ __forceinline__ void mg_issue_C(const MgArgs &a, const MgLayer *, int l, int cta, uint8_t *dst, uint64_t *bar,
                                           uint64_t pol) {
	if (cta >= a.C.units) return;
	mg_issue(dst, a.tiled + size_t(l) * a.tl_layer + a.tl_C + size_t(cta) * a.C.bytes, a.C.bytes, bar, pol);
}
__device__ __forceinline__ void mg_issue_D(const MgArgs &a, const MgLayer *, int l, int cta, uint8_t *dst, uint64_t *bar,
                                           uint64_t pol) {
	if (cta >= a.Dp.units) return;
	mg_issue(dst, a.tiled + size_t(l) * a.tl_layer + a.tl_D + size_t(cta) * a.Dp.bytes, a.Dp.bytes, bar, pol);
}
__device__ __forceinline__ void mg_issue_E(const MgArgs &a, const MgLayer *, int l, int cta, uint8_t *dst, uint64_t *bar,
                                           uint64_t pol) {
	if (cta >= a.E.units) return;
	mg_issue(dst, a.tiled + size_t(l) * a.tl_layer + a.tl_E + size_t(cta) * a.E.bytes, a.E.bytes, bar, pol);
}

// Copy `ntiles_mat` column tiles x `nsplit` K-splits of a row-major int8 matrix [K][N] into unit
// order: unit (split, tile0 + t) becomes a contiguous [kc][TN] block at
// dst + (split * ntiles_total + tile0 + t) * unit_stride + dst_off. One thread per 16 bytes.
__global__ void retile_kernel(int8_t *dst, const int8_t *src, int N, int TN, int kc, int nsplit, int ntiles_total, int tile0,
                              int ntiles_mat, size_t unit_stride, size_t dst_off) {
	const int segs = TN / 16;
	const size_t total = size_t(nsplit) * ntiles_mat * kc * segs;
	for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
		const int seg = int(i % segs);
		const int r = int((i / segs) % kc);
		const int t = int((i / (size_t(segs) * kc)) % ntiles_mat);
		const int split = int(i / (size_t(segs) * kc * ntiles_mat));
		const int4 v = *reinterpret_cast<const int4 *>(src + size_t(split * kc + r) * N + t * TN + seg * 16);
		*reinterpret_cast<int4 *>(dst + size_t(split * ntiles_total + tile0 + t) * unit_stride + dst_off + (size_t(r) * segs + seg) * 16) = v;
	}
}



// Per-thread slices (d = tid, tid+384, tid+768) of the three D-long vectors a
// residual+norm prologue needs. They are cold in DRAM (read once per token),
// so they are loaded into registers BEFORE the grid barrier that precedes the
// prologue and are there when the barrier opens.
// Norm weights and column scales of a residual+norm prologue, held in registers:
// thread t < D/4 owns elements 4t..4t+3 of every D-vector.
struct MgVec3 {
	float4 s, wpost, wpre;
};
__device__ __forceinline__ void mg_load_vec3(MgVec3 &v, const float *scale, const float *w_post, const float *w_pre, int D) {
	const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
	const int t = threadIdx.x;
	const bool in = 4 * t < D;
	v.s = (in && scale) ? __ldg(reinterpret_cast<const float4 *>(scale) + t) : z;
	v.wpost = (in && w_post) ? __ldg(reinterpret_cast<const float4 *>(w_post) + t) : z;
	v.wpre = (in && w_pre) ? __ldg(reinterpret_cast<const float4 *>(w_pre) + t) : z;
}

// If has_t: t[d] = scale[d] * sum_s part[s][d];  h += rmsnorm(t; w_post).
// Then xs[0..D) = rmsnorm(h; w_pre). Every CTA computes the same bits.
// D <= 4 * MG_THREADS, D % 4 == 0. The partial sums of all splits are requested
// at once so that the L2 round trips overlap; with `ll` they are polled until
// complete (self-validating hand-off), otherwise they are plain loads behind a
// grid barrier. Splits are added in ascending order.
__device__ __noinline__ void mg_resnorm(const MgArgs &a, MgCtx &c, float *h, float *xs, float *bred, bool has_t,
                                        const float *part, int nsplit, bool ll, const MgVec3 v, float *x_out,
                                        unsigned tag = 0, int n_pres = 0) {
	const int D = a.D, tid = threadIdx.x;
	const bool in = 4 * tid < D;
	float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
	if (in) hv = *reinterpret_cast<const float4 *>(h + 4 * tid);  // own elements: written by this thread
	if (has_t) {
		float4 tv = make_float4(0.f, 0.f, 0.f, 0.f);
		if (!ll) {
			// tagged words {value, tag}: `part` is the layer's buffer of uint2, [nsplit][D] followed by
			// n_pres presence words (CTAs without a unit of the producing phase); threads past D/4 poll those
			const uint2 *pe = reinterpret_cast<const uint2 *>(part);
#pragma unroll 1
			for (int s0 = 0; s0 < nsplit; s0 += 4) {
				uint4 w[4][2];
				int spins = 0;
				bool ok;
				do {
					ok = true;
#pragma unroll
					for (int q = 0; q < 4; q++) {
						w[q][0] = w[q][1] = make_uint4(0u, tag, 0u, tag);
						if (in && s0 + q < nsplit) {
							const uint2 *src = pe + size_t(s0 + q) * D + 4 * tid;
							w[q][0] = ld_tagged2(src);
							w[q][1] = ld_tagged2(src + 2);
						}
					}
					if (s0 == 0 && !in && tid - D / 4 < n_pres)
						ok = ld_tagged_acquire(pe + size_t(nsplit) * D + (tid - D / 4)).y == tag;
#pragma unroll
					for (int q = 0; q < 4; q++)
						ok = ok && w[q][0].y == tag && w[q][0].w == tag && w[q][1].y == tag && w[q][1].w == tag;
				} while (!ok && ll_retry(c, spins));
#pragma unroll
				for (int q = 0; q < 4; q++) {
					tv.x += __uint_as_float(w[q][0].x);
					tv.y += __uint_as_float(w[q][0].z);
					tv.z += __uint_as_float(w[q][1].x);
					tv.w += __uint_as_float(w[q][1].z);
				}
			}
		}
#pragma unroll 1
		for (int s0 = 0; ll && s0 < nsplit; s0 += 8) {
			float4 pv[8];
			int spins = 0;
			bool ok;
			do {
				ok = true;
#pragma unroll
				for (int q = 0; q < 8; q++) {
					pv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
					if (in && s0 + q < nsplit) {
						const float *src = part + size_t(s0 + q) * D + 4 * tid;
						pv[q] = ll_load4_once(src);
					}
				}
#pragma unroll
				for (int q = 0; q < 8; q++) ok = ok && ll_valid(pv[q]);
			} while (!ok && ll_retry(c, spins));
#pragma unroll
			for (int q = 0; q < 8; q++) {
				tv.x += pv[q].x;
				tv.y += pv[q].y;
				tv.z += pv[q].z;
				tv.w += pv[q].w;
			}
		}
		tv.x *= v.s.x;
		tv.y *= v.s.y;
		tv.z *= v.s.z;
		tv.w *= v.s.w;
		float ss = fmaf(tv.x, tv.x, fmaf(tv.y, tv.y, fmaf(tv.z, tv.z, tv.w * tv.w)));
		ss = mg_block_sum<MG_NWARPS>(ss, bred);
		const float r1 = inv_rms(ss, D);
		hv.x = hv.x + (tv.x * r1) * (v.wpost.x + 1.0f);
		hv.y = hv.y + (tv.y * r1) * (v.wpost.y + 1.0f);
		hv.z = hv.z + (tv.z * r1) * (v.wpost.z + 1.0f);
		hv.w = hv.w + (tv.w * r1) * (v.wpost.w + 1.0f);
		if (in) *reinterpret_cast<float4 *>(h + 4 * tid) = hv;
	}
	float ss2 = fmaf(hv.x, hv.x, fmaf(hv.y, hv.y, fmaf(hv.z, hv.z, hv.w * hv.w)));
	ss2 = mg_block_sum<MG_NWARPS>(ss2, bred);
	const float r2 = inv_rms(ss2, D);
	if (in) {
		float4 y;
		y.x = (hv.x * r2) * (v.wpre.x + 1.0f);
		y.y = (hv.y * r2) * (v.wpre.y + 1.0f);
		y.z = (hv.z * r2) * (v.wpre.z + 1.0f);
		y.w = (hv.w * r2) * (v.wpre.w + 1.0f);
		*reinterpret_cast<float4 *>(xs + 4 * tid) = y;
		if (x_out) *reinterpret_cast<float4 *>(x_out + 4 * tid) = y;
	}
	__syncthreads();
}

// Phase C prologue: merge the attention partials for rows k0..k0+kc of the head-major output
// into xs[0..kc). Kept out of line so that its registers do not add to the layer loop's.
__device__ __noinline__ void mg_attn_merge(const MgArgs &a, MgCtx &ctx, const float *attn_part, int nsA, int k0, float *att,
                                           float *red, float *xs) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	// Merge the attention partials for rows k0..k0+kc of the head-major output:
	// o = sum_s w[s][h] * o_s with w = exp(m_s - M) / sum_s l_s exp(m_s - M).
	// Thread -> (16-byte piece of the row range, group of partials); every load is in
	// flight before the first wait, and the partials are polled until complete.
	float *sml = att;                   // [nsA][8]: m[4], l[4] of every partial
	float *wgt = att + 8 * MG_MAX_ATT;  // [nsA][4]
	const int kc4 = a.C.kc / 4;
	const int ngrp = max(1, MG_THREADS / kc4);
	const int per = (nsA + ngrp - 1) / ngrp;  // partials per group
	const int grp = tid / kc4, c4 = tid - grp * kc4;
	const bool worker = grp < ngrp;
	const int sp0 = grp * per, sp1 = min(nsA, sp0 + per);
	// stage 1: the (m, l) words of every partial. They are small, so CTAs that idle through the
	// attention phase poll these and leave the L2 to the attention CTAs.
	{
		float4 mlv = make_float4(0.f, 0.f, 0.f, 0.f);
		const float *mlp = attn_part + size_t(tid >> 1) * (AT_NH * AT_HD + 8) + AT_NH * AT_HD + 4 * (tid & 1);
		int spins = 0;
		if (tid < 2 * nsA) {
			do {
				mlv = ll_load4_once(mlp);
			} while (!ll_valid(mlv) && ll_retry(ctx, spins));
			*reinterpret_cast<float4 *>(sml + (tid >> 1) * 8 + 4 * (tid & 1)) = mlv;
		}
	}
	__syncthreads();
	if (warp < AT_NH) {  // warp = head; lanes stride over the partials
		float M = -INFINITY;
#pragma unroll 1
		for (int sp = lane; sp < nsA; sp += 32) M = fmaxf(M, sml[sp * 8 + warp]);
		M = warp_max(M);
		float Ls = 0.0f;
#pragma unroll 1
		for (int sp = lane; sp < nsA; sp += 32) {
			const float ms = sml[sp * 8 + warp];
			const float ee = (ms == -INFINITY) ? 0.0f : expf(ms - M);
			wgt[sp * 4 + warp] = ee;
			Ls = fmaf(sml[sp * 8 + 4 + warp], ee, Ls);
		}
		Ls = warp_sum(Ls);
		const float inv = 1.0f / Ls;
#pragma unroll 1
		for (int sp = lane; sp < nsA; sp += 32) wgt[sp * 4 + warp] *= inv;
	}
	// stage 2: the partial outputs, eight 16-byte pieces in flight per thread
	float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
	const int eh = (k0 + 4 * c4) / AT_HD;
	float4 ov[8];
	auto load_batch = [&](int s0) {
		int spins = 0;
		bool ok;
		do {
			ok = true;
#pragma unroll
			for (int q = 0; q < 8; q++) {
				ov[q] = make_float4(0.f, 0.f, 0.f, 0.f);
				if (worker && s0 + q < sp1) ov[q] = ll_load4_once(attn_part + size_t(s0 + q) * (AT_NH * AT_HD + 8) + k0 + 4 * c4);
			}
#pragma unroll
			for (int q = 0; q < 8; q++) ok = ok && ll_valid(ov[q]);
		} while (!ok && ll_retry(ctx, spins));
	};
	load_batch(sp0);
	__syncthreads();  // the weights are ready
#pragma unroll 1
	for (int s0 = sp0; s0 < sp1; s0 += 8) {
		if (s0 > sp0) load_batch(s0);
#pragma unroll
		for (int q = 0; q < 8; q++) {
			if (worker && s0 + q < sp1) {
				const float w = wgt[(s0 + q) * 4 + eh];
				acc.x = fmaf(ov[q].x, w, acc.x);
				acc.y = fmaf(ov[q].y, w, acc.y);
				acc.z = fmaf(ov[q].z, w, acc.z);
				acc.w = fmaf(ov[q].w, w, acc.w);
			}
		}
	}
	if (worker) *reinterpret_cast<float4 *>(red + grp * a.C.kc + 4 * c4) = acc;
	__syncthreads();
#pragma unroll 1
	for (int d = tid; d < a.C.kc; d += MG_THREADS) {  // (a K-slice of two heads has more rows than the CTA has threads)
		float O = 0.0f;
#pragma unroll 1
		for (int g = 0; g < ngrp; g++) O += red[g * a.C.kc + d];
		xs[d] = O;
	}
	__syncthreads();

}

__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok)
	    : "r"(smem_u32(bar)), "r"(parity)
	    : "memory");
	return ok != 0;
}
#define MG_STAMP()                                                   \
	do {                                                             \
		if (dbg_on && dbg_n < a.dbg_cap) a.dbg[dbg_n++] = clock64(); \
	} while (0)

__global__ void __launch_bounds__(MG_THREADS, 1) mega_decode_kernel(const __grid_constant__ MgArgs a) {
	extern __shared__ uint8_t smem_raw[];
	uint8_t *smem = reinterpret_cast<uint8_t *>((uintptr_t(smem_raw) + 1023) & ~uintptr_t(1023));
	__shared__ uint64_t bar_A, bar_C, bar_D, bar_E, bar_lm[MG_LM_STAGES], emp_lm[MG_LM_STAGES];
	__shared__ float bred[MG_NWARPS];
	__shared__ int s_abort;
	__shared__ float s_f[8];
	__shared__ int s_i[4];
	__shared__ int s_cdf[2 * MG_NWARPS + 8];
	__shared__ float wm[3][AT_NH], wl[3][AT_NH];
	__shared__ MgLayer s_ly[MG_MAX_LAYERS];

	uint8_t *R_A = smem + a.off_A, *R_C = smem + a.off_C, *R_D = smem + a.off_D, *R_E = smem + a.off_E;
	float *h = reinterpret_cast<float *>(smem + a.off_h);
	float *xs = reinterpret_cast<float *>(smem + a.off_xs);
	float *red = reinterpret_cast<float *>(smem + a.off_red);
	float *att = reinterpret_cast<float *>(smem + a.off_att);  // qs[4][256] | ks[256] | vs[256]
	float *qs = att, *ks = att + AT_NH * AT_HD, *vs = ks + AT_HD;

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x;
	const int D = a.D, L = a.L;
	const int NQ = a.QD + 2 * a.KD;

	if (tid == 0) {
		mbar_init(&bar_A, 1);
		mbar_init(&bar_C, 1);
		mbar_init(&bar_D, 1);
		mbar_init(&bar_E, 1);
#pragma unroll 1
		for (int i = 0; i < MG_LM_STAGES; i++) {
			mbar_init(&bar_lm[i], 1);
			mbar_init(&emp_lm[i], MG_NWARPS);
		}
		s_abort = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	{
		const int *src = reinterpret_cast<const int *>(a.layers);
		int *dst = reinterpret_cast<int *>(s_ly);
#pragma unroll 1
		for (int i = tid; i < L * int(sizeof(MgLayer) / 4); i += MG_THREADS) dst[i] = src[i];
	}
	__syncthreads();
	MgCtx ctx{&s_abort, a.err, a.bar, 0u, unsigned(G)};
	uint32_t pA = 0, pC = 0, pD = 0, pE = 0, plm = 0, pemp = 0;  // phase parities (plm, pemp: one bit per ring stage)
	const uint64_t pol = l2_evict_first_policy();

	if (warp == 0) {
		mg_issue_A(a, s_ly, 0, cta, R_A, &bar_A, pol);
		mg_issue_C(a, s_ly, 0, cta, R_C, &bar_C, pol);
		mg_issue_D(a, s_ly, 0, cta, R_D, &bar_D, pol);
		mg_issue_E(a, s_ly, 0, cta, R_E, &bar_E, pol);
	}

	int tok = __ldcg(a.tok);
	int pos = __ldcg(a.next_pos);
	const int rbase = __ldcg(a.ring_base);
	int n_logged = 0;
	int dbg_n = 0;
	MgVec3 vA;  // vectors for the next residual+norm prologue of phase A / lm_head
	mg_load_vec3(vA, nullptr, nullptr, s_ly[0].attn_pre, D);

#pragma unroll 1
	for (int step = 0; step < a.n_steps; step++) {
		const bool more = (step + 1 < a.n_steps);
		const bool dbg_on = (a.dbg != nullptr) && cta == a.dbg_cta && tid == 0 && !more;
		MG_STAMP();
		// ---------------------------------------------------------------- embedding
		if (tok < 0 || tok >= a.V) {
			if (tid == 0 && cta == 0) atomicExch(a.err, 1);
			tok = 0;
		}
#pragma unroll 1
		for (int d = tid; d < D; d += MG_THREADS) h[d] = a.wte_s[d] * (a.sqrtD * float(a.wte[size_t(tok) * D + d]));
		__syncthreads();

#pragma unroll 1
		for (int l = 0; l < L; l++) {
			const MgLayer &ly = s_ly[l];
			const int nsA = ly.is_local ? a.att_local : a.att_global;
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
			const int chunk = (valid + nsA - 1) / nsA;
			const int j0 = cta * chunk, j1 = min(valid, j0 + chunk);
			// Hand-off buffers of this layer (one of two copies; the other copy is wiped below for
			// the next layer — its readers all passed the grid barrier that ended the previous layer).
			const int lc = step * L + l;
			float *const llb = a.ll + size_t(lc & 1) * a.ll_stride;
#define part_A (llb + a.ll_pA)
#define attn_part (llb + a.ll_att)
#define part_C (llb + a.ll_pC)
#define act (llb + a.ll_act)
			// down projection -> next layer hand-off: tagged words, buffer and tag follow the launch-spanning layer count
			const unsigned gl = a.seq0 + unsigned(lc);
#define pe_cur (a.pe + size_t(gl & 1u) * a.pe_stride)
#define pe_prev (a.pe + size_t((gl & 1u) ^ 1u) * a.pe_stride)
			const int n_pres = G - a.E.units;
			// ============================================================ A: QKV
			float4 qsc = make_float4(0.f, 0.f, 0.f, 0.f);  // scales of this thread's 4 q|k|v columns (attention CTAs)
			{
				const bool active = cta < a.A.units;
				const int tile = active ? cta % a.A.ntiles : 0, split = active ? cta / a.A.ntiles : 0;
				const int k0 = split * a.A.kc;
				mg_resnorm(a, ctx, h, xs, bred, l > 0, reinterpret_cast<const float *>(pe_prev), a.E.nsplit, false, vA, nullptr, gl, n_pres);
				if (warp == 1 && l > 0 && (a.sched & 2)) mg_issue_E(a, s_ly, l, cta, R_E, &bar_E, pol);
				MG_STAMP();
				if (active) mg_wait_tma(ctx, &bar_A, pA);
				MG_STAMP();
				if (active) {
					const float s = mg_tile_colsum(R_A, a.A.kc, a.A, xs + k0, red);
					// q, k, v tiles are consecutive and equally wide: tile -> column of the q|k|v vector
					if (tid < a.A.TN) ll_store(part_A + size_t(split) * NQ + tile * a.A.TN + tid, s);
				}
				pA ^= 1;
				MG_STAMP();
				__syncthreads();  // R_A is free again
				if (warp == 1) {
					if (l + 1 < L)
						mg_issue_A(a, s_ly, l + 1, cta, R_A, &bar_A, pol);
					else if (more)
						mg_issue_A(a, s_ly, 0, cta, R_A, &bar_A, pol);
				}
				// Wipe the other copy of the hand-off arena (last used by the previous layer, next used by
				// the next one). Every CTA has finished reading it: this CTA got past the prologue above,
				// which needs the down-projection words (or presence word) of ALL CTAs, and those are
				// stored after the storing CTA's last read of the previous layer's buffers. The CTAs that
				// idle through the attention phase do the wiping; the fence orders it before their own
				// next down-projection / presence store, which is what lets anyone write that copy again.
				if (cta >= nsA) {
					float4 *other = reinterpret_cast<float4 *>(a.ll + size_t((lc & 1) ^ 1) * a.ll_stride);
					const int nw = G - nsA, n4 = a.ll_stride / 4, per = (n4 + nw - 1) / nw;
					const float e = __uint_as_float(MG_LL_EMPTY);
#pragma unroll 1
					for (int i = (cta - nsA) * per + tid; i < min(n4, (cta - nsA + 1) * per); i += MG_THREADS)
						__stcg(other + i, make_float4(e, e, e, e));
					__syncthreads();
					if (tid == 0) __threadfence();
				}
				// cold data of phase B
				if (cta < nsA) {
					if (4 * tid < NQ) {
						const int n = 4 * tid;
						const float *sp = n < a.QD ? ly.sq + n : (n < a.QD + a.KD ? ly.sk + (n - a.QD) : ly.sv + (n - a.QD - a.KD));
						qsc = __ldg(reinterpret_cast<const float4 *>(sp));
					}
					const float *cosr = a.rope[ly.is_local][0] + size_t(p) * AT_HD;
					const float *sinr = a.rope[ly.is_local][1] + size_t(p) * AT_HD;
					if (tid < 8) {
						prefetch_l2(cosr + 32 * tid);
						prefetch_l2(sinr + 32 * tid);
						prefetch_l2(ly.rmsq + 32 * tid);
						prefetch_l2(ly.rmsk + 32 * tid);
					}
					// this CTA's cache rows: 1 KiB per row = 8 lines, K and V
#pragma unroll 1
					for (int i = tid; i < (j1 - j0) * 8; i += MG_THREADS) {
						prefetch_l2(ly.kcache + size_t(j0) * AT_HD + 32 * i);
						prefetch_l2(ly.vcache + size_t(j0) * AT_HD + 32 * i);
					}
				}
				MG_STAMP();
			}
			// ============================================================ B: attention
			{
				if (cta < nsA) {
					// q|k|v = scale * sum of K-split partials (polled: phase A's CTAs store them as they finish)
					float *qkv = red;  // NQ floats; `red` is free here
					if (4 * tid < NQ) {
						float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
						for (int s0 = 0; s0 < a.A.nsplit; s0 += 8) {
							float4 pv[8];
							int spins = 0;
							bool ok;
							do {
								ok = true;
#pragma unroll
								for (int q = 0; q < 8; q++) {
									pv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
									if (s0 + q < a.A.nsplit) pv[q] = ll_load4_once(part_A + size_t(s0 + q) * NQ + 4 * tid);
								}
#pragma unroll
								for (int q = 0; q < 8; q++) ok = ok && ll_valid(pv[q]);
							} while (!ok && ll_retry(ctx, spins));
#pragma unroll
							for (int q = 0; q < 8; q++) {
								sum.x += pv[q].x;
								sum.y += pv[q].y;
								sum.z += pv[q].z;
								sum.w += pv[q].w;
							}
						}
						*reinterpret_cast<float4 *>(qkv + 4 * tid) =
						    make_float4(sum.x * qsc.x, sum.y * qsc.y, sum.z * qsc.z, sum.w * qsc.w);
					}
					__syncthreads();
					const float *cosr = a.rope[ly.is_local][0] + size_t(p) * AT_HD;
					const float *sinr = a.rope[ly.is_local][1] + size_t(p) * AT_HD;
					if (warp < AT_NH)
						norm_rope_head(qkv + warp * AT_HD, ly.rmsq, cosr, sinr, 0.0625f, qs + warp * AT_HD);
					else if (warp == AT_NH)
						norm_rope_head(qkv + AT_NH * AT_HD, ly.rmsk, cosr, sinr, 1.0f, ks);
					else if (warp == AT_NH + 1)
#pragma unroll 1
						for (int d = lane; d < AT_HD; d += 32) vs[d] = qkv[AT_NH * AT_HD + AT_HD + d];
					__syncthreads();
					if (slot >= j0 && slot < j1) {
#pragma unroll 1
						for (int d = tid; d < AT_HD; d += MG_THREADS) {
							ly.kcache[size_t(slot) * AT_HD + d] = ks[d];
							ly.vcache[size_t(slot) * AT_HD + d] = vs[d];
						}
					}
					// warp -> (head, key group): 4 heads x 3 groups; lane owns dims 4*lane..+3 and 128+4*lane..+3
					const int hh = warp & 3, grp = warp >> 2;
					const float4 q0 = *reinterpret_cast<const float4 *>(qs + hh * AT_HD + 4 * lane);
					const float4 q1 = *reinterpret_cast<const float4 *>(qs + hh * AT_HD + 128 + 4 * lane);
					float4 o0 = make_float4(0.f, 0.f, 0.f, 0.f), o1 = make_float4(0.f, 0.f, 0.f, 0.f);
					float m = -INFINITY, lsum = 0.0f;
#pragma unroll 1
					for (int jb = j0 + grp; jb < j1; jb += 9) {
						float4 kv[3][4];
						bool live[3];
#pragma unroll
						for (int u = 0; u < 3; u++) {
							const int j = jb + 3 * u;
							live[u] = j < j1;
							if (!live[u]) continue;
							if (j == slot) {
								kv[u][0] = *reinterpret_cast<const float4 *>(ks + 4 * lane);
								kv[u][1] = *reinterpret_cast<const float4 *>(ks + 128 + 4 * lane);
								kv[u][2] = *reinterpret_cast<const float4 *>(vs + 4 * lane);
								kv[u][3] = *reinterpret_cast<const float4 *>(vs + 128 + 4 * lane);
							} else {
								const float *kr = ly.kcache + size_t(j) * AT_HD, *vr = ly.vcache + size_t(j) * AT_HD;
								kv[u][0] = __ldcg(reinterpret_cast<const float4 *>(kr + 4 * lane));
								kv[u][1] = __ldcg(reinterpret_cast<const float4 *>(kr + 128 + 4 * lane));
								kv[u][2] = __ldcg(reinterpret_cast<const float4 *>(vr + 4 * lane));
								kv[u][3] = __ldcg(reinterpret_cast<const float4 *>(vr + 128 + 4 * lane));
							}
						}
#pragma unroll
						for (int u = 0; u < 3; u++) {
							if (!live[u]) continue;
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
					}
					// merge the 3 key groups of every head through `red` ([3][4][256] floats)
					if (lane == 0) {
						wm[grp][hh] = m;
						wl[grp][hh] = lsum;
					}
					*reinterpret_cast<float4 *>(red + (grp * AT_NH + hh) * AT_HD + 4 * lane) = o0;
					*reinterpret_cast<float4 *>(red + (grp * AT_NH + hh) * AT_HD + 128 + 4 * lane) = o1;
					__syncthreads();
					float *prow = attn_part + size_t(cta) * (AT_NH * AT_HD + 8);
#pragma unroll 1
					for (int e = tid; e < AT_NH * AT_HD; e += MG_THREADS) {
						const int eh = e / AT_HD;
						const float M = fmaxf(fmaxf(wm[0][eh], wm[1][eh]), wm[2][eh]);
						float Ls = 0.0f, O = 0.0f;
#pragma unroll
						for (int g = 0; g < 3; g++) {
							const float ee = (wm[g][eh] == -INFINITY) ? 0.0f : expf(wm[g][eh] - M);
							Ls = fmaf(wl[g][eh], ee, Ls);
							O = fmaf(red[(g * AT_NH + eh) * AT_HD + (e % AT_HD)], ee, O);
						}
						ll_store(prow + e, O);
						if ((e % AT_HD) == 0) {
							ll_store(prow + AT_NH * AT_HD + eh, M);
							ll_store(prow + AT_NH * AT_HD + 4 + eh, Ls);
						}
					}
					__syncthreads();  // `red`, `att` are reused by phase C
				}
				MG_STAMP();
			}
			// ============================================================ C: O projection
			MgVec3 vD;       // vectors of phase D's residual+norm prologue
			float su_r = 0.0f, sg_r = 0.0f;  // scales of this thread's up/gate column
			{
				const bool active = cta < a.C.units;
				const int tile = active ? cta % a.C.ntiles : 0, split = active ? cta / a.C.ntiles : 0;
				const int k0 = split * a.C.kc;
				if (active) {
					mg_attn_merge(a, ctx, attn_part, nsA, k0, att, red, xs);
				}
				MG_STAMP();
				if (active) {
					mg_wait_tma(ctx, &bar_C, pC);
					const float s = mg_tile_colsum(R_C, a.C.kc, a.C, xs, red);
					if (tid < a.C.TN) ll_store(part_C + size_t(split) * D + tile * a.C.TN + tid, s);
				}
				pC ^= 1;
				MG_STAMP();
				__syncthreads();  // R_C is free again
				if (warp == 1) {
					if (l + 1 < L)
						mg_issue_C(a, s_ly, l + 1, cta, R_C, &bar_C, pol);
					else if (more)
						mg_issue_C(a, s_ly, 0, cta, R_C, &bar_C, pol);
				}
				mg_load_vec3(vD, ly.so, ly.attn_post, ly.mlp_pre, D);
				if (cta < a.Dp.units && tid < a.Dp.TN) {
					su_r = __ldg(ly.su + cta * a.Dp.TN + tid);
					sg_r = __ldg(ly.sg + cta * a.Dp.TN + tid);
				}
				MG_STAMP();
			}
			// ============================================================ D: up & gate + GeGLU
			{
				const bool active = cta < a.Dp.units;
				mg_resnorm(a, ctx, h, xs, bred, true, part_C, a.C.nsplit, true, vD, nullptr);
				MG_STAMP();
				if (active) mg_wait_tma(ctx, &bar_D, pD);
				MG_STAMP();
				float up = 0.0f;
				if (active) up = mg_tile_colsum(R_D, D, a.Dp, xs, red);
				MG_STAMP();
				if (active) {
					const float gate = mg_tile_colsum(R_D + a.Dp.TN * D, D, a.Dp, xs, red);
					if (tid < a.Dp.TN) ll_store(act + cta * a.Dp.TN + tid, a.lut(gate * sg_r) * (up * su_r));
				}
				pD ^= 1;
				MG_STAMP();
				__syncthreads();  // R_D is free again
				if (warp == 1 && l + 1 < L && !(a.sched & 1)) mg_issue_D(a, s_ly, l + 1, cta, R_D, &bar_D, pol);
				MG_STAMP();
			}
			// ============================================================ E: down projection
			{
				const bool active = cta < a.E.units;
				const int tile = active ? cta % a.E.ntiles : 0, split = active ? cta / a.E.ntiles : 0;
				const int k0 = split * a.E.kc;
				if (active) {
					// this CTA's rows of the activation vector, polled until complete
					const int n4 = a.E.kc / 4;
#pragma unroll 1
					for (int i0 = 0; i0 < n4; i0 += 5 * MG_THREADS) {
						float4 v[5];
						int spins = 0;
						bool ok;
						do {
							ok = true;
#pragma unroll
							for (int q = 0; q < 5; q++) {
								const int i = i0 + q * MG_THREADS + tid;
								v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
								if (i < n4) v[q] = ll_load4_once(act + k0 + 4 * i);
							}
#pragma unroll
							for (int q = 0; q < 5; q++) ok = ok && ll_valid(v[q]);
						} while (!ok && ll_retry(ctx, spins));
#pragma unroll
						for (int q = 0; q < 5; q++) {
							const int i = i0 + q * MG_THREADS + tid;
							if (i < n4) *reinterpret_cast<float4 *>(xs + 4 * i) = v[q];
						}
					}
					__syncthreads();
					mg_wait_tma(ctx, &bar_E, pE);
				}
				if (warp == 1 && l + 1 < L && (a.sched & 1)) mg_issue_D(a, s_ly, l + 1, cta, R_D, &bar_D, pol);
				MG_STAMP();
				if (active) {
					const float s = mg_tile_colsum(R_E, a.E.kc, a.E, xs, red);
					if (tid < a.E.TN) st_tagged(pe_cur + size_t(split) * D + tile * a.E.TN + tid, s, gl + 1u);
				}
				pE ^= 1;
				MG_STAMP();
				// a CTA without a unit still reports that it is done reading this layer's hand-off buffers
				if (!active && tid == 0) st_tagged(pe_cur + size_t(a.E.nsplit) * D + (cta - a.E.units), 0.0f, gl + 1u);
				if (warp == 1 && l + 1 < L && !(a.sched & 2)) mg_issue_E(a, s_ly, l + 1, cta, R_E, &bar_E, pol);
				if (l + 1 < L)
					mg_load_vec3(vA, ly.sd, ly.mlp_post, s_ly[l + 1].attn_pre, D);
				else
					mg_load_vec3(vA, ly.sd, ly.mlp_post, a.final_norm, D);
				MG_STAMP();
			}
#undef part_A
#undef attn_part
#undef part_C
#undef act
#undef pe_cur
#undef pe_prev
		}

		// ================================================================ lm_head
		// logits[v] = lm_scale[v] * sum_k x[k] W[k,v]; this CTA takes column tiles
		// cta, cta+G, ...; a tile's K rows stream through a ring of MG_LM_STAGES
		// stages of LM.box_rows rows laid over the (now idle) D and E regions.
		{
			const unsigned gl_last = a.seq0 + unsigned(step * L + L - 1);
			mg_resnorm(a, ctx, h, xs, bred, true, reinterpret_cast<const float *>(a.pe + size_t(gl_last & 1u) * a.pe_stride),
			           a.E.nsplit, false, vA, cta == 0 ? a.xnorm_out : nullptr, gl_last + 1u, G - a.E.units);
		}
		MG_STAMP();
		float best = -INFINITY;  // running max of this CTA's (temperature-scaled) logits, threads < 128
		int best_i = -1;
		{
			// Ring protocol: full[stage] completes when the TMA bytes have landed; each of the
			// 12 warps arrives on empty[stage] when it has read the stage; one lane then refills
			// it. No block-wide barrier per chunk — only the tile-end reduction synchronises.
			const MgPhase &ph = a.LM;
			const int bps = a.lm_bps;                 // boxes per stage
			const int spt = ph.nboxes / bps;          // stages per column tile
			const int stage_rows = ph.box_rows * bps;
			const int my_tiles = (ph.ntiles - cta + G - 1) / G;
			const int total = my_tiles * spt;  // stages this CTA consumes
			const int box_bytes = ph.TN * ph.box_rows;
			const int stage_bytes = box_bytes * bps;
			uint8_t *ring = R_D;
			auto issue_stage = [&](int q, int stg) {  // by one lane
				const int t = cta + (q / spt) * G, c = q % spt;
				mbar_expect_tx(&bar_lm[stg], uint32_t(stage_bytes));
				for (int b = 0; b < bps; b++)
					tma_load_2d(ring + stg * stage_bytes + b * box_bytes, a.tmaps + a.tm_lm, t * ph.TN,
					            c * stage_rows + b * ph.box_rows, &bar_lm[stg], pol);
			};
			if (warp == MG_NWARPS - 1) {
				if (lane == 0) fence_proxy_async();
				__syncwarp();
				if (lane < MG_LM_STAGES && lane < total) issue_stage(lane, lane);
			}
			float acc[16];
			float sc_tile = 0.0f;
			const int rstep = ph.rstep;
			const int row0 = ph.segs == 1 ? tid : int(__umulhi(tid, ph.m_segs));
			int stg = 0, c = 0, tile = cta;  // ring stage, stage within the tile, column tile: advanced at the loop's end
#pragma unroll 1
			for (int q = 0; q < total; q++) {
				if (c == 0) {
#pragma unroll
					for (int i = 0; i < 16; i++) acc[i] = 0.0f;
					if (tid < ph.TN) sc_tile = __ldg(a.lm_scale + tile * ph.TN + tid);  // cold: ask early
				}
				mg_wait_tma(ctx, &bar_lm[stg], (plm >> stg) & 1u);
				plm ^= (1u << stg);
				{
					const uint8_t *tp = ring + stg * stage_bytes + 16 * tid;
					const float *xc = xs + c * stage_rows;
					int row = row0;
#pragma unroll 1
					for (; row + 3 * rstep < stage_rows; row += 4 * rstep) {
						int4 v0 = *reinterpret_cast<const int4 *>(tp);
						int4 v1 = *reinterpret_cast<const int4 *>(tp + 16 * MG_THREADS);
						int4 v2 = *reinterpret_cast<const int4 *>(tp + 32 * MG_THREADS);
						int4 v3 = *reinterpret_cast<const int4 *>(tp + 48 * MG_THREADS);
						const float x0 = xc[row], x1 = xc[row + rstep], x2 = xc[row + 2 * rstep], x3 = xc[row + 3 * rstep];
						tp += 64 * MG_THREADS;
						mg_fma16(acc, v0, x0);
						mg_fma16(acc, v1, x1);
						mg_fma16(acc, v2, x2);
						mg_fma16(acc, v3, x3);
					}
#pragma unroll 1
					for (; row < stage_rows; row += rstep) {
						int4 v = *reinterpret_cast<const int4 *>(tp);
						tp += 16 * MG_THREADS;
						mg_fma16(acc, v, xc[row]);
					}
				}
				__syncwarp();
				if (lane == 0) mbar_arrive(&emp_lm[stg]);
				if (warp == MG_NWARPS - 1 && lane == 0) {
					const int nq = q + MG_LM_STAGES;
					if (nq < total) {
						mg_wait_tma(ctx, &emp_lm[stg], (pemp >> stg) & 1u);  // all 12 warps have left the stage
						fence_proxy_async();
						issue_stage(nq, stg);
					}
				}
				pemp ^= (1u << stg);
				__syncwarp();
				if (c == spt - 1) {
					float s = mg_tile_reduce(acc, ph, red);
					if (tid < ph.TN) {
						const int v = tile * ph.TN + tid;
						const float lg = s * sc_tile;
						__stcg(a.logits + v, lg);
						const float z = (a.sampler == 2) ? lg / a.temp : lg;
						if (z > best) {  // tiles ascend, so the first maximum keeps the lowest index
							best = z;
							best_i = v;
						}
					}
				}
				if (++stg == MG_LM_STAGES) stg = 0;
				if (++c == spt) {
					c = 0;
					tile += G;
				}
			}
		}
		__syncthreads();

		// ================================================================ sampler
		MG_STAMP();
		int next_tok = 0;
		if (a.sampler == 0) {
			mg_grid_sync(ctx);  // logits complete
		} else {
			// CTA-local (max, argmax): value descending, index ascending; index -1 never beats a real one
			auto better = [](float v1, int i1, float v2, int i2) {
				if (v1 > v2) return true;
				if (v1 < v2) return false;
				if (i2 < 0) return i1 >= 0;
				if (i1 < 0) return false;
				return i1 < i2;
			};
			if (tid < 128) {
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
					s_f[warp] = best;
					s_i[warp] = best_i;
				}
			}
			__syncthreads();
			if (tid == 0) {
				for (int w = 1; w < 4; w++)
					if (better(s_f[w], s_i[w], best, best_i)) {
						best = s_f[w];
						best_i = s_i[w];
					}
				__stcg(a.samp_f + cta, best);
				__stcg(a.samp_i + cta, best_i);
			}
			mg_grid_sync(ctx);
			// every CTA reduces the per-CTA results the same way (warp 0, 5 batched loads per lane)
			if (warp == 0) {
				float gv[8];
				int gi[8];
#pragma unroll
				for (int q = 0; q < 8; q++) {
					const int c = lane + 32 * q;
					gv[q] = c < G ? __ldcg(a.samp_f + c) : -INFINITY;
					gi[q] = c < G ? __ldcg(a.samp_i + c) : -1;
				}
				float gmax = gv[0];
				int gidx = gi[0];
#pragma unroll
				for (int q = 1; q < 8; q++)
					if (better(gv[q], gi[q], gmax, gidx)) {
						gmax = gv[q];
						gidx = gi[q];
					}
#pragma unroll 1
				for (int c = lane + 256; c < G; c += 32) {
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
					const int my_tiles = (a.LM.ntiles - cta + G - 1) / G;
#pragma unroll 1
					for (int j = tid; j < my_tiles * MG_LM_TN; j += MG_THREADS) {
						const int v = (cta + (j / MG_LM_TN) * G) * MG_LM_TN + (j % MG_LM_TN);
						const float pv = expf(__ldcg(a.logits + v) / a.temp - gmax);
						__stcg(a.probs + v, pv);
						ds += (pv < cut) ? 0.0f : pv;
					}
				}
				ds = mg_block_sum<MG_NWARPS>(ds, bred);
				if (tid == 0) __stcg(a.samp_f + G + cta, ds);
				mg_grid_sync(ctx);
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
					float *cbuf = reinterpret_cast<float *>(R_D);
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
						for (int i = tid * 4; i < n; i += MG_THREADS * 4) {
							float4 v = __ldcg(reinterpret_cast<const float4 *>(a.probs + c0 + i));
							v.x *= inv;
							v.y *= inv;
							v.z *= inv;
							v.w *= inv;
							*reinterpret_cast<float4 *>(cbuf + i) = v;
						}
						__syncthreads();
						const int r = cdf_cross_block<MG_NWARPS>(cbuf, n, &s_f[5], randf, s_cdf, c0 == 0 ? 1024 : 0);
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
				mg_grid_sync(ctx);
				next_tok = __ldcg(a.samp_i + G);
			}
			if (cta == 0 && tid == 0) {
				if (a.tok_log && n_logged < a.log_cap) a.tok_log[n_logged] = next_tok;
				*a.tok = next_tok;
			}
			n_logged++;
		}
		MG_STAMP();
		pos += 1;
		if (cta == 0 && tid == 0) *a.next_pos = pos;
		// the ring is idle again: fetch the next token's layer-0 up/gate and down tiles
		if (warp == 0 && more) {
			mg_issue_D(a, s_ly, 0, cta, R_D, &bar_D, pol);
			mg_issue_E(a, s_ly, 0, cta, R_E, &bar_E, pol);
		}
		if (more) mg_load_vec3(vA, nullptr, nullptr, s_ly[0].attn_pre, D);
		tok = next_tok;
		if (*(volatile int *)&s_abort) break;
	}
	if (cta == 0 && tid == 0 && a.log_count) *a.log_count = n_logged;
}

}  // namespace tg
