// On-device samplers over the 262144-way logits row of each sequence.
#pragma once
#include "tg_common.cuh"

namespace tg {

constexpr int SM_THREADS = 1024;
constexpr int SM_NWARPS = SM_THREADS / 32;

struct SampleArgs {
	float *logits;   // [B][V]; min-p overwrites it with the reference's "probabilities"
	int V;
	int *tok_out;    // [B] token fed to the next decode step
	int *tok_log;    // [max_steps][B] or null
	int *log_count;  // [B] entries written so far per sequence (device counter)
	int log_cap;     // capacity in steps
	int B;
	// min-p
	float minp, temp;
	const float *randf;  // [n][B] uniforms, indexed by randf_count[b]
	int *randf_count;    // [B]
	int randf_cap;
};

__device__ __forceinline__ void emit_token(const SampleArgs &a, int b, int tok) {
	a.tok_out[b] = tok;
	if (a.tok_log) {
		int c = a.log_count[b];
		if (c < a.log_cap) a.tok_log[size_t(c) * a.B + b] = tok;
		a.log_count[b] = c + 1;
	}
}

// ops::argmax_logits, reference ops.hpp:744-760: ascending scan with a strict
// '>' — the lowest index wins ties, NaN never wins, -1 if nothing exceeds -inf.
__global__ void __launch_bounds__(SM_THREADS) argmax_kernel(SampleArgs a) {
	pdl_trigger();
	pdl_wait();
	__shared__ float sv[SM_NWARPS];
	__shared__ int si[SM_NWARPS];
	const int b = blockIdx.x, tid = threadIdx.x;
	const float *x = a.logits + size_t(b) * a.V;
	float best = -INFINITY;
	int arg = -1;
	for (int i = tid * 4; i < a.V; i += SM_THREADS * 4) {
		float4 v = __ldcg(reinterpret_cast<const float4 *>(x + i));
		if (v.x > best) { best = v.x; arg = i; }
		if (v.y > best) { best = v.y; arg = i + 1; }
		if (v.z > best) { best = v.z; arg = i + 2; }
		if (v.w > best) { best = v.w; arg = i + 3; }
	}
	// (value desc, index asc); arg == -1 loses to any real index at equal value
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
		int oi = __shfl_xor_sync(0xffffffffu, arg, o);
		if (better(ov, oi, best, arg)) { best = ov; arg = oi; }
	}
	if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = arg; }
	__syncthreads();
	if (tid == 0) {
		for (int w = 1; w < SM_NWARPS; w++)
			if (better(sv[w], si[w], best, arg)) { best = sv[w]; arg = si[w]; }
		emit_token(a, b, arg);
	}
}

// ------------------------------------------------------------------ exact parallel inverse CDF
// Step (6) of min-p sampling is "the first index whose running fp32 sum reaches randf", where the
// running sum is the sequential chain cum = fl(cum + p[i]). fp32 addition is not associative, so a
// tree sum would move the crossing index. The chain can still be evaluated in parallel, exactly:
// while cum stays in one binade [2^e, 2^(e+1)) it is an integer multiple S of u = 2^(e-23), and
// adding p rounds S + p/u to the nearest integer, ties to even. So element i acts on S as
//     S -> S + a0[i]  (S even),   S -> S + a1[i]  (S odd),
// with a0 = a1 = round(p/u) except on an exact tie, where the pair encodes round-half-even. Such
// maps compose into maps of the same form (the parity of the result follows from the parity of the
// input), so a prefix scan of (a0, a1) pairs gives every partial sum of the chain, bit for bit.
// When a sum would leave the binade, that one addition is done in fp32 and the scan restarts behind
// it with the new u. Sums saturate far above every threshold, so they stay monotone.
struct CdfFn {
	int a0, a1;
};
constexpr int CDF_SAT = 1 << 27;
constexpr int CDF_BIG = 1 << 25;
__device__ __forceinline__ CdfFn cdf_compose(CdfFn f, CdfFn g) {  // first f, then g
	CdfFn h;
	h.a0 = min(CDF_SAT, f.a0 + ((f.a0 & 1) ? g.a1 : g.a0));
	h.a1 = min(CDF_SAT, f.a1 + ((f.a1 & 1) ? g.a0 : g.a1));
	return h;
}
__device__ __forceinline__ int cdf_apply(CdfFn f, int S) { return min(CDF_SAT, S + ((S & 1) ? f.a1 : f.a0)); }
__device__ __forceinline__ CdfFn cdf_element(float p, float inv_u) {
	const float x = p * inv_u;
	CdfFn f;
	if (!(x < 33554432.0f)) {  // also NaN / inf: forces the fp32 path for this element
		f.a0 = f.a1 = CDF_BIG;
		return f;
	}
	const float fl = floorf(x);
	const float fr = x - fl;  // exact
	const int q = int(fl);
	if (fr == 0.5f) {
		f.a0 = q + (q & 1);
		f.a1 = q + 1 - (q & 1);
	} else {
		f.a0 = f.a1 = q + (fr > 0.5f ? 1 : 0);
	}
	return f;
}

constexpr int CDF_PER_LANE = 8;
constexpr int CDF_PER_WARP = 32 * CDF_PER_LANE;

// Block-cooperative (NW warps, all threads call it with the same arguments). p[0..n) lies in shared
// memory; *cum_io (shared) holds the running sum before p[0] and receives the sum after the last
// element consumed. Returns the first index i with fl(cum + p[0] + ... + p[i]) >= randf, or -1.
// scratch: 2 * NW + 8 ints of shared memory.
// The first elements of a row are added one by one by a single thread: the running sum starts at
// zero and changes binade about log2(position) times, and every change would cost a whole scan
// round (≈ 1 us, the time of ≈ 400 sequential additions). p >= 0, so the sum never decreases and
// a group of 8 is searched only when its last partial sum has reached randf.
__device__ __forceinline__ void cdf_cross_seq(const float *p, int end, float randf, float &cum, int &pos, int &res) {
	float c = cum;
	int i = pos;
	for (; i + 8 <= end; i += 8) {
		const float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
		float cs[8];
		cs[0] = c + a.x;
		cs[1] = cs[0] + a.y;
		cs[2] = cs[1] + a.z;
		cs[3] = cs[2] + a.w;
		cs[4] = cs[3] + b.x;
		cs[5] = cs[4] + b.y;
		cs[6] = cs[5] + b.z;
		cs[7] = cs[6] + b.w;
		if (cs[7] >= randf) {
			int k = 7;
#pragma unroll
			for (int t = 6; t >= 0; t--)
				if (cs[t] >= randf) k = t;
			res = i + k;
			cum = cs[k];
			pos = i + k + 1;
			return;
		}
		c = cs[7];
	}
	for (; i < end; i++) {
		c += p[i];
		if (c >= randf) {
			res = i;
			cum = c;
			pos = i + 1;
			return;
		}
	}
	cum = c;
	pos = i;
}

// `seq_limit`: leading elements that one thread adds sequentially (see cdf_cross_seq) before the
// block-wide scan takes over; pass ~1000 for the start of a row, 0 for later chunks. p must be
// 16-byte aligned.
template <int NW>
__device__ int cdf_cross_block(const float *p, int n, float *cum_io, float randf, int *scratch, int seq_limit = 0) {
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	CdfFn *wt = reinterpret_cast<CdfFn *>(scratch);  // per-warp composite
	int *s_pos = scratch + 2 * NW, *s_res = scratch + 2 * NW + 1;
	if (tid == 0) {
		float cum = *cum_io;
		int pos = 0, res = -1;
		if (seq_limit > 0) cdf_cross_seq(p, min(n, seq_limit), randf, cum, pos, res);
		*cum_io = cum;
		*s_pos = pos;
		*s_res = res;
	}
	__syncthreads();
	for (int guard = 0; guard < n + 64; guard++) {  // every round consumes at least one element
		const int pos = *s_pos;
		if (*s_res >= 0 || pos >= n) break;
		const float cum = *cum_io;
		const unsigned bits = __float_as_uint(cum);
		const int e = int((bits >> 23) & 0xffu) - 127;
		if (!(cum >= 7.888609e-31f) || e > 120) {
			// zero, tiny, inf or NaN: plain fp32 steps until the sum is an ordinary number
			__syncthreads();
			if (tid == 0) {
				float c = cum;
				int i = pos, r = -1;
				for (; i < n && r < 0; i++) {
					c += p[i];
					if (c >= randf) r = i;
					if (c >= 7.888609e-31f && c < 1e36f) {
						i++;
						break;
					}
				}
				*cum_io = c;
				*s_pos = i;
				*s_res = r;
			}
			__syncthreads();
			continue;
		}
		const float u = __uint_as_float(unsigned(e - 23 + 127) << 23);
		const float inv_u = __uint_as_float(unsigned(23 - e + 127) << 23);
		const int S0 = int(cum * inv_u);
		const float y = randf * inv_u;
		const int T = (y < 33554432.0f) ? int(ceilf(y)) : CDF_BIG;
		const int Tmin = min(T, 1 << 24);
		// this lane's elements
		const int base = pos + warp * CDF_PER_WARP + lane * CDF_PER_LANE;
		CdfFn el[CDF_PER_LANE];
		CdfFn mine{0, 0};
#pragma unroll
		for (int k = 0; k < CDF_PER_LANE; k++) {
			el[k] = CdfFn{0, 0};
			if (base + k < n) el[k] = cdf_element(p[base + k], inv_u);
			mine = cdf_compose(mine, el[k]);
		}
		// inclusive scan over the lanes
		CdfFn inc = mine;
#pragma unroll
		for (int o = 1; o < 32; o <<= 1) {
			CdfFn prev;
			prev.a0 = __shfl_up_sync(0xffffffffu, inc.a0, o);
			prev.a1 = __shfl_up_sync(0xffffffffu, inc.a1, o);
			if (lane >= o) inc = cdf_compose(prev, inc);
		}
		if (lane == 31) wt[warp] = inc;
		CdfFn exc;
		exc.a0 = __shfl_up_sync(0xffffffffu, inc.a0, 1);
		exc.a1 = __shfl_up_sync(0xffffffffu, inc.a1, 1);
		if (lane == 0) exc = CdfFn{0, 0};
		__syncthreads();
		// state at the start of every warp; first warp in which the sum reaches the threshold
		int Sw = S0, hit = -1, Shit = 0;
#pragma unroll 1
		for (int w = 0; w < NW; w++) {
			const int nx = cdf_apply(wt[w], Sw);
			if (hit < 0 && nx >= Tmin) {
				hit = w;
				Shit = Sw;
			}
			Sw = nx;
		}
		__syncthreads();  // wt is rewritten next round
		if (hit < 0) {
			if (tid == 0) {
				*cum_io = float(Sw) * u;  // exact: Sw < 2^24
				*s_pos = pos + NW * CDF_PER_WARP;
			}
		} else if (warp == hit) {
			int S = cdf_apply(exc, Shit);
			int jfirst = -1, Sbefore = 0, Safter = 0;
#pragma unroll
			for (int k = 0; k < CDF_PER_LANE; k++) {
				const int nx = cdf_apply(el[k], S);
				if (jfirst < 0 && nx >= Tmin) {
					jfirst = base + k;
					Sbefore = S;
					Safter = nx;
				}
				S = nx;
			}
			const unsigned m = __ballot_sync(0xffffffffu, jfirst >= 0);
			const int src = __ffs(m) - 1;  // m != 0: this warp's total reaches the threshold
			if (lane == src) {
				if (Safter < (1 << 24)) {
					*s_res = jfirst;  // the sum reached randf inside the binade
					*cum_io = float(Safter) * u;
					*s_pos = jfirst + 1;
				} else {
					const float c = float(Sbefore) * u + p[jfirst];  // the one addition that leaves the binade
					*cum_io = c;
					*s_pos = jfirst + 1;
					if (c >= randf) *s_res = jfirst;
				}
			}
		}
		__syncthreads();
	}
	__syncthreads();
	return *s_res;
}

// ops::minp_logits, reference ops.hpp:762-859.
//  (1) x /= temp  (2) rowmax  (3) p = exp(x - rowmax), maxp  (4) cut = minp*maxp,
//  denom = sum of p >= cut  (5) every p *= 1/denom — tokens under the cut keep
//  their mass, only the denominator is masked  (6) first index whose running
//  fp32 sum reaches randf, else 0.
// Steps 1-5 are data-parallel. Step 6 must reproduce a *sequential* fp32 sum
// (fp32 addition is not associative, and the crossing index depends on the
// rounding): cdf_cross_block evaluates that chain exactly, in parallel, over
// chunks that the whole CTA stages into shared memory.
constexpr int MP_CHUNK = 8192;

__global__ void __launch_bounds__(SM_THREADS) minp_kernel(SampleArgs a) {
	__shared__ float red[SM_NWARPS];
	__shared__ float chunk[MP_CHUNK];
	__shared__ int scratch[2 * SM_NWARPS + 8];
	__shared__ float s_cum;
	const int b = blockIdx.x, tid = threadIdx.x;
	float *x = a.logits + size_t(b) * a.V;
	float randf = 0.0f;
	{
		int rc = a.randf_count[b];
		if (rc < a.randf_cap) randf = a.randf[size_t(rc) * a.B + b];
	}
	// (1)+(2)
	float mx = -INFINITY;
	for (int i = tid * 4; i < a.V; i += SM_THREADS * 4) {
		float4 v = __ldcg(reinterpret_cast<const float4 *>(x + i));
		v.x = v.x / a.temp; v.y = v.y / a.temp; v.z = v.z / a.temp; v.w = v.w / a.temp;
		__stcg(reinterpret_cast<float4 *>(x + i), v);
		mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
	}
	mx = warp_max(mx);
	if ((tid & 31) == 0) red[tid >> 5] = mx;
	__syncthreads();
	float rowmax = -INFINITY;
	for (int w = 0; w < SM_NWARPS; w++) rowmax = fmaxf(rowmax, red[w]);
	__syncthreads();
	// (3)
	float mp = -INFINITY;
	for (int i = tid * 4; i < a.V; i += SM_THREADS * 4) {
		float4 v = __ldcg(reinterpret_cast<const float4 *>(x + i));
		v.x = expf(v.x - rowmax); v.y = expf(v.y - rowmax); v.z = expf(v.z - rowmax); v.w = expf(v.w - rowmax);
		__stcg(reinterpret_cast<float4 *>(x + i), v);
		mp = fmaxf(mp, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
	}
	mp = warp_max(mp);
	if ((tid & 31) == 0) red[tid >> 5] = mp;
	__syncthreads();
	float maxp = -INFINITY;
	for (int w = 0; w < SM_NWARPS; w++) maxp = fmaxf(maxp, red[w]);
	__syncthreads();
	// (4)
	const float cut = a.minp * maxp;
	float ds = 0.0f;
	for (int i = tid * 4; i < a.V; i += SM_THREADS * 4) {
		float4 v = __ldcg(reinterpret_cast<const float4 *>(x + i));
		ds += (v.x < cut) ? 0.0f : v.x;
		ds += (v.y < cut) ? 0.0f : v.y;
		ds += (v.z < cut) ? 0.0f : v.z;
		ds += (v.w < cut) ? 0.0f : v.w;
	}
	ds = warp_sum(ds);
	if ((tid & 31) == 0) red[tid >> 5] = ds;
	__syncthreads();
	float denom = 0.0f;
	for (int w = 0; w < SM_NWARPS; w++) denom += red[w];
	const float inv = 1.0f / denom;
	// (5)+(6): every chunk is scaled (the reference scales the whole row); the running sum is
	// evaluated chunk by chunk until the crossing is known
	if (tid == 0) s_cum = 0.0f;
	__syncthreads();
	int found = -1;
	for (int c0 = 0; c0 < a.V; c0 += MP_CHUNK) {
		const int n = min(MP_CHUNK, a.V - c0);
		for (int i = tid * 4; i < n; i += SM_THREADS * 4) {
			float4 v = __ldcg(reinterpret_cast<const float4 *>(x + c0 + i));
			v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
			__stcg(reinterpret_cast<float4 *>(x + c0 + i), v);
			*reinterpret_cast<float4 *>(&chunk[i]) = v;
		}
		__syncthreads();
		if (found < 0) {
			const int r = cdf_cross_block<SM_NWARPS>(chunk, n, &s_cum, randf, scratch, c0 == 0 ? 1024 : 0);
			if (r >= 0) found = c0 + r;
		}
		__syncthreads();
	}
	if (tid == 0) {
		emit_token(a, b, found < 0 ? 0 : found);
		a.randf_count[b] += 1;
	}
}


// ------------------------------------------------------------------ grid-wide min-p (one sequence)
// ops::minp_logits for a single row spread over G CTAs of SG_THREADS threads (cooperative launch: the
// CTAs meet at a bounded grid barrier). It partitions the row and orders every floating-point sum
// exactly like the sampler inside the persistent decode kernel — CTA c owns the 128-column tiles
// c, c + G, ...; per-thread strided sums, a 12-warp block sum, the G partial sums added by one warp
// in lane-strided order — so a token sampled step by step (tg_decode + tg_sample_minp) is the token
// the device-resident loop samples. The row is overwritten with the probabilities, as the
// reference does.
constexpr int SG_THREADS = 384;
constexpr int SG_NWARPS = SG_THREADS / 32;
constexpr int SG_TILE = 128;
constexpr int SG_SPIN_CAP = 1 << 22;

__device__ __forceinline__ bool sg_grid_sync(unsigned *bar, unsigned &epoch, unsigned G, int *fail) {
	__syncthreads();
	epoch += 1;
	if (threadIdx.x == 0 && !*(volatile int *)fail) {
		__threadfence();
		const unsigned old = atomicAdd(bar, 1u);
		if (old + 1u < epoch * G) {
			int spins = 0;
			unsigned v;
			do {
				asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
			} while (v < epoch * G && ++spins < SG_SPIN_CAP);
			if (v < epoch * G) *fail = 1;  // the wait ran out: everybody falls through from here on
		}
	}
	__syncthreads();
	return !*(volatile int *)fail;
}

template <int NW>
__device__ __forceinline__ float sg_block_sum(float v, float *red) {
	v = warp_sum(v);
	__syncthreads();
	if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
	__syncthreads();
	float t = 0.0f;
#pragma unroll
	for (int w = 0; w < NW; w++) t += red[w];
	return t;
}

// part: [2 * G] floats of scratch, probs: [V] floats of scratch, bar: one zeroed word, err: error word
__global__ void __launch_bounds__(SG_THREADS, 1) minp_grid_kernel(SampleArgs a, unsigned *bar, float *part, float *probs, int *err) {
	__shared__ float red[SG_NWARPS];
	__shared__ float chunk[MP_CHUNK];
	__shared__ int scratch[2 * SG_NWARPS + 8];
	__shared__ float s_cum, s_inv, s_max;
	__shared__ int s_fail, s_tok;
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x;
	const int ntiles = a.V / SG_TILE;
	const int my_tiles = (ntiles - cta + G - 1) / G;
	unsigned epoch = 0;
	if (tid == 0) s_fail = 0;
	__syncthreads();
	// (1)+(2) row maximum of z = logit / temp
	float mx = -INFINITY;
#pragma unroll 1
	for (int j = tid; j < my_tiles * SG_TILE; j += SG_THREADS) {
		const int v = (cta + (j / SG_TILE) * G) * SG_TILE + (j % SG_TILE);
		mx = fmaxf(mx, __ldcg(a.logits + v) / a.temp);
	}
	mx = warp_max(mx);
	if (lane == 0) red[warp] = mx;
	__syncthreads();
	if (tid == 0) {
		float m = red[0];
		for (int w = 1; w < SG_NWARPS; w++) m = fmaxf(m, red[w]);
		__stcg(part + cta, m);
	}
	sg_grid_sync(bar, epoch, G, &s_fail);
	if (warp == 0) {
		float m = -INFINITY;
#pragma unroll 1
		for (int c = lane; c < G; c += 32) m = fmaxf(m, __ldcg(part + c));
		m = warp_max(m);
		if (lane == 0) s_max = m;
	}
	__syncthreads();
	const float gmax = s_max;
	// (3)+(4) p = exp(z - max); maxp = exp(0), so the cut is minp * exp(gmax - gmax); masked denominator
	const float cut = a.minp * expf(gmax - gmax);
	float ds = 0.0f;
#pragma unroll 1
	for (int j = tid; j < my_tiles * SG_TILE; j += SG_THREADS) {
		const int v = (cta + (j / SG_TILE) * G) * SG_TILE + (j % SG_TILE);
		const float pv = expf(__ldcg(a.logits + v) / a.temp - gmax);
		__stcg(probs + v, pv);
		ds += (pv < cut) ? 0.0f : pv;
	}
	ds = sg_block_sum<SG_NWARPS>(ds, red);
	if (tid == 0) __stcg(part + G + cta, ds);
	sg_grid_sync(bar, epoch, G, &s_fail);
	if (warp == 0) {
		float dv = 0.0f;
#pragma unroll 1
		for (int c = lane; c < G; c += 32) dv += __ldcg(part + G + c);
		dv = warp_sum(dv);
		if (lane == 0) s_inv = 1.0f / dv;
	}
	__syncthreads();
	const float inv = s_inv;
	// (5) every probability is scaled in place of its logit
#pragma unroll 1
	for (int j = tid; j < my_tiles * SG_TILE; j += SG_THREADS) {
		const int v = (cta + (j / SG_TILE) * G) * SG_TILE + (j % SG_TILE);
		__stcg(a.logits + v, __ldcg(probs + v) * inv);
	}
	// (6) inverse CDF by CTA 0
	if (cta == 0 && !*(volatile int *)&s_fail) {
		float randf = 0.0f;
		const int rc = a.randf_count[0];
		if (rc < a.randf_cap) randf = a.randf[size_t(rc) * a.B];
		if (tid == 0) {
			s_cum = 0.0f;
			s_tok = -1;
		}
		__syncthreads();
#pragma unroll 1
		for (int c0 = 0; c0 < a.V; c0 += MP_CHUNK) {
			const int n = min(MP_CHUNK, a.V - c0);
#pragma unroll 4
			for (int i = tid * 4; i < n; i += SG_THREADS * 4) {
				float4 v = __ldcg(reinterpret_cast<const float4 *>(probs + c0 + i));
				v.x *= inv;
				v.y *= inv;
				v.z *= inv;
				v.w *= inv;
				*reinterpret_cast<float4 *>(chunk + i) = v;
			}
			__syncthreads();
			const int r = cdf_cross_block<SG_NWARPS>(chunk, n, &s_cum, randf, scratch, c0 == 0 ? 1024 : 0);
			if (r >= 0) {
				if (tid == 0) s_tok = c0 + r;
				break;
			}
		}
		__syncthreads();
		if (tid == 0) {
			emit_token(a, 0, s_tok < 0 ? 0 : s_tok);
			a.randf_count[0] = rc + 1;
		}
	}
	if (tid == 0 && *(volatile int *)&s_fail) atomicExch(err, 8);
}

// The inverse-CDF step in isolation over an explicit vector p[0..n) in global memory, starting
// from the running sum cum0: *idx = first i with fl(cum0 + p[0] + ... + p[i]) >= randf, else -1.
// One CTA; *cum_out receives the sum after the last element consumed.
__global__ void __launch_bounds__(SM_THREADS) inverse_cdf_kernel(const float *p, int n, float cum0, float randf, int *idx,
                                                                 float *cum_out) {
	__shared__ float chunk[MP_CHUNK];
	__shared__ int scratch[2 * SM_NWARPS + 8];
	__shared__ float s_cum;
	const int tid = threadIdx.x;
	if (tid == 0) s_cum = cum0;
	__syncthreads();
	int found = -1;
	for (int c0 = 0; c0 < n && found < 0; c0 += MP_CHUNK) {
		const int m = min(MP_CHUNK, n - c0);
		for (int i = tid; i < m; i += SM_THREADS) chunk[i] = p[c0 + i];
		__syncthreads();
		const int r = cdf_cross_block<SM_NWARPS>(chunk, m, &s_cum, randf, scratch, c0 == 0 ? 1024 : 0);
		if (r >= 0) found = c0 + r;
		__syncthreads();
	}
	if (tid == 0) {
		*idx = found;
		*cum_out = s_cum;
	}
}

}  // namespace tg
