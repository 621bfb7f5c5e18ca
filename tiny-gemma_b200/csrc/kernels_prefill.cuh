// Prefill kernels: many tokens of one sequence at a time. Row-wise norms,
// the int8-weight GEMM on CUDA cores (fp32 FMA), q/k norm + RoPE + cache fill,
// causal / sliding-window attention over the prompt, GeGLU.
#pragma once
#include "tg_common.cuh"

namespace tg {

// ops::embedding_prefill, reference ops.hpp:529-571
__global__ void embed_prefill_kernel(const int8_t *wte, const float *scales, const int *ids, float *h, int S, int D,
                                     int V, float sqrtD, int *err_flag) {
	pdl_trigger();
	pdl_wait();
	int s = blockIdx.x;
	int tok = ids[s];
	if (tok < 0 || tok >= V) {
		if (threadIdx.x == 0) *err_flag = 1;
		tok = 0;
	}
	const int8_t *row = wte + size_t(tok) * D;
	for (int d = threadIdx.x; d < D; d += blockDim.x) h[size_t(s) * D + d] = scales[d] * (sqrtD * float(row[d]));
}

// out[s,:] = (res ? res[s,:] : 0) + rmsnorm(in[s,:]; w). One CTA of 256 threads
// per row. ops::rmsnorm (+ ops::add), reference ops.hpp:126-222, 84-103.
// `out` may alias `res` or `in`.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(float *out, const float *in, const float *w, const float *res,
                                                            int dim) {
	pdl_trigger();
	pdl_wait();
	__shared__ float bred[8];
	const size_t off = size_t(blockIdx.x) * dim;
	float ss = 0.0f;
	for (int d = threadIdx.x; d < dim; d += 256) {
		float v = in[off + d];
		ss = fmaf(v, v, ss);
	}
	ss = block_sum<8>(ss, bred);
	const float r = inv_rms(ss, dim);
	for (int d = threadIdx.x; d < dim; d += 256) {
		float y = (in[off + d] * r) * (w[d] + 1.0f);
		out[off + d] = res ? (res[off + d] + y) : y;
	}
}

// ---------------------------------------------------------------- GEMM (CUDA cores)
// C[M,N] = scale[n] * sum_k A[m,k] * W[k,n]   (gemm::qgemmnn, reference linalg.hpp:210-308)
// 64x128 output tile per CTA, K stepped by 32; W converted int8->fp32 once per
// tile on its way into shared memory; each of 256 threads owns a 4x8 block.
// Optional split along K (grid.z) with partials summed by a second kernel.
constexpr int GM_BM = 64, GM_BN = 128, GM_BK = 32;

__global__ void __launch_bounds__(256) qgemm_simt_kernel(float *C, const float *A, const int8_t *W, const float *scales,
                                                         int M, int K, int N, int kc, float *partial) {
	__shared__ __align__(16) float As[GM_BK][GM_BM + 4];
	__shared__ __align__(16) float Ws[GM_BK][GM_BN];
	const int tid = threadIdx.x;
	const int n0 = blockIdx.x * GM_BN, m0 = blockIdx.y * GM_BM;
	const int kbeg = blockIdx.z * kc, kend = min(K, kbeg + kc);
	const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads: rows 4*ty.., cols 8*tx..
	float acc[4][8];
#pragma unroll
	for (int i = 0; i < 4; i++)
#pragma unroll
		for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

	for (int kk = kbeg; kk < kend; kk += GM_BK) {
		// A tile: 64 rows x 32 k -> As[k][m]; thread loads 8 floats (2 float4)
#pragma unroll
		for (int r = 0; r < 2; r++) {
			int idx = tid + r * 256;        // 0..511 float4 slots
			int m = idx >> 3, k4 = idx & 7;  // 64 rows x 8 float4
			float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
			if (m0 + m < M) v = *reinterpret_cast<const float4 *>(A + size_t(m0 + m) * K + kk + 4 * k4);
			As[4 * k4 + 0][m] = v.x;
			As[4 * k4 + 1][m] = v.y;
			As[4 * k4 + 2][m] = v.z;
			As[4 * k4 + 3][m] = v.w;
		}
		// W tile: 32 k x 128 cols int8 = 256 int4 -> one per thread
		{
			int k = tid >> 3, c16 = tid & 7;
			int4 v = ld_stream_int4(W + size_t(kk + k) * N + n0 + 16 * c16);
			const uint32_t words[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
#pragma unroll
			for (int j = 0; j < 4; j++) {
				float f[4];
				i8x4_to_f32(words[j], f);
				*reinterpret_cast<float4 *>(&Ws[k][16 * c16 + 4 * j]) = make_float4(f[0], f[1], f[2], f[3]);
			}
		}
		__syncthreads();
#pragma unroll
		for (int k = 0; k < GM_BK; k++) {
			float4 a4 = *reinterpret_cast<const float4 *>(&As[k][4 * ty]);
			float4 w0 = *reinterpret_cast<const float4 *>(&Ws[k][8 * tx]);
			float4 w1 = *reinterpret_cast<const float4 *>(&Ws[k][8 * tx + 4]);
			const float av[4] = {a4.x, a4.y, a4.z, a4.w};
			const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
			for (int i = 0; i < 4; i++)
#pragma unroll
				for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 4; i++) {
		int m = m0 + 4 * ty + i;
		if (m >= M) continue;
		if (gridDim.z == 1) {
#pragma unroll
			for (int j = 0; j < 8; j++) C[size_t(m) * N + n0 + 8 * tx + j] = acc[i][j] * scales[n0 + 8 * tx + j];
		} else {
			float *p = partial + (size_t(blockIdx.z) * M + m) * N + n0 + 8 * tx;
#pragma unroll
			for (int j = 0; j < 8; j++) p[j] = acc[i][j];
		}
	}
}

__global__ void qgemm_splitk_reduce_kernel(float *C, const float *partial, const float *scales, int M, int N, int nsplit,
                                           int ldc) {
	size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= size_t(M) * N) return;
	float s = 0.0f;
	for (int sp = 0; sp < nsplit; sp++) s += partial[size_t(sp) * M * N + i];
	const size_t m = i / N, n = i % N;
	C[m * ldc + n] = s * scales[n];
}

// the same for a launch over up to three matrices (columns col0[g] .. of a partial-sum row belong to group g)
struct ReduceGroups {
	int ngroups;
	int col0[4];  // col0[ngroups] = total columns
	const float *scales[3];
	float *C[3];
	int ldc[3];
};
__global__ void qgemm_splitk_reduce_groups_kernel(ReduceGroups g, const float *partial, int M, int N, int nsplit) {
	size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= size_t(M) * N) return;
	float s = 0.0f;
	for (int sp = 0; sp < nsplit; sp++) s += partial[size_t(sp) * M * N + i];
	const size_t m = i / N;
	const int n = int(i % N);
	// (selects over constant indices: indexing the parameter arrays with a run-time value would move them to local memory)
	const int gi = (n >= g.col0[1] && g.ngroups > 1) + (n >= g.col0[2] && g.ngroups > 2);
	const int c0 = gi == 0 ? g.col0[0] : (gi == 1 ? g.col0[1] : g.col0[2]);
	float *Cp = gi == 0 ? g.C[0] : (gi == 1 ? g.C[1] : g.C[2]);
	const float *sp_ = gi == 0 ? g.scales[0] : (gi == 1 ? g.scales[1] : g.scales[2]);
	const int ld = gi == 0 ? g.ldc[0] : (gi == 1 ? g.ldc[1] : g.ldc[2]);
	const int nl = n - c0;
	Cp[m * ld + nl] = s * sp_[nl];
}

// out[b, :] = table lookup per element: gate = lut(gate) * up over [rows][n] with row strides
// (the batched decode step keeps up and gate in separate buffers)

// ops::gelu (LUT) + ops::mul, reference ops.hpp:62-123: gate = lut(gate) * up
__global__ void geglu_kernel(float *gate, const float *up, size_t n, GeluLut lut) {
	size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i < n) gate[i] = lut(gate[i]) * up[i];
}

// q/k per-head RMSNorm + RoPE at position s (offset 0) in place on
// q [S][4*256] and k [S][256], and KVCache::update_prefill (reference
// decode.hpp:72-105): the last min(S, slots) prompt positions go to cache
// slots 0.. in order. One CTA (5 warps + 1) per prompt position.
// With nsplit > 0 the projections arrive as the raw K-split partial sums of the grouped q|k|v GEMM
// (part[(sp * S + s) * 1536 + n], columns q | k | v) with the column scales sq / sk / sv; the splits are
// added in ascending order and scaled here, and v is written out as well.
// Several prompts of the same length share a launch: blockIdx.y is the prompt, its rows are
// blockIdx.y * S .. of the `rows` rows of q / k / v / part, and its caches follow each other at
// cache_stride floats.
__global__ void __launch_bounds__(192) qk_norm_rope_prefill_kernel(float *q, float *k, float *v, const float *rmsq,
                                                                    const float *rmsk, const float *cosT,
                                                                    const float *sinT, float *kcache, float *vcache,
                                                                    int S, int slots, const float *part, int nsplit,
                                                                    const float *sq, const float *sk, const float *sv,
                                                                    int rows, size_t cache_stride) {
	pdl_trigger();
	pdl_wait();
	const int s = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	{
		const size_t r0 = size_t(blockIdx.y) * S;  // first row of this prompt
		q += r0 * 1024;
		k += r0 * 256;
		v += r0 * 256;
		if (part) part += r0 * 1536;
		kcache += blockIdx.y * cache_stride;
		vcache += blockIdx.y * cache_stride;
	}
	const float *cosr = cosT + size_t(s) * 256, *sinr = sinT + size_t(s) * 256;
	const int start = (S >= slots) ? (S - slots) : 0;
	const int c = s - start;  // cache slot, if >= 0
	// raw element n of this position's q|k|v row (n = column in the concatenated 1536), scaled by scale[ns]
	auto raw = [&](int n, const float *scale, int ns) -> float {
		return sum_splits(part + size_t(s) * 1536 + n, size_t(rows) * 1536, nsplit) * scale[ns];
	};
	// x: the head's 256 floats (finished projection if nsplit == 0; always the destination)
	auto norm_rope = [&](float *x, const float *w, int n0, const float *scale, int ns0) {
		float lo[4], hi[4];
		float ss = 0.0f;
		if (nsplit > 0) {
			// the lane's eight elements x four splits are requested together; splits are added in ascending order
#pragma unroll
			for (int i = 0; i < 4; i++) lo[i] = hi[i] = 0.0f;
			const size_t sstride = size_t(rows) * 1536;
			const float *base = part + size_t(s) * 1536 + n0 + 4 * lane;
			for (int s0 = 0; s0 < nsplit; s0 += 4) {
				float4 a[4], b[4];
#pragma unroll
				for (int q = 0; q < 4; q++) {
					a[q] = b[q] = make_float4(0.f, 0.f, 0.f, 0.f);
					if (s0 + q < nsplit) {
						a[q] = *reinterpret_cast<const float4 *>(base + size_t(s0 + q) * sstride);
						b[q] = *reinterpret_cast<const float4 *>(base + size_t(s0 + q) * sstride + 128);
					}
				}
#pragma unroll
				for (int q = 0; q < 4; q++) {
					lo[0] += a[q].x; lo[1] += a[q].y; lo[2] += a[q].z; lo[3] += a[q].w;
					hi[0] += b[q].x; hi[1] += b[q].y; hi[2] += b[q].z; hi[3] += b[q].w;
				}
			}
#pragma unroll
			for (int i = 0; i < 4; i++) {
				lo[i] *= scale[ns0 + 4 * lane + i];
				hi[i] *= scale[ns0 + 128 + 4 * lane + i];
			}
		} else {
#pragma unroll
			for (int i = 0; i < 4; i++) {
				lo[i] = x[4 * lane + i];
				hi[i] = x[128 + 4 * lane + i];
			}
		}
#pragma unroll
		for (int i = 0; i < 4; i++) {
			ss = fmaf(lo[i], lo[i], ss);
			ss = fmaf(hi[i], hi[i], ss);
		}
		ss = warp_sum(ss);
		const float r = inv_rms(ss, 256);
#pragma unroll
		for (int i = 0; i < 4; i++) {
			const int d = 4 * lane + i;
			float a = (lo[i] * r) * (w[d] + 1.0f);
			float b = (hi[i] * r) * (w[d + 128] + 1.0f);
			x[d] = fmaf(-1.0f * b, sinr[d], cosr[d] * a);
			x[d + 128] = fmaf(a, sinr[d + 128], cosr[d + 128] * b);
		}
	};
	if (warp < 4) {
		norm_rope(q + size_t(s) * 1024 + warp * 256, rmsq, warp * 256, sq, warp * 256);
	} else if (warp == 4) {
		float *kr = k + size_t(s) * 256;
		norm_rope(kr, rmsk, 1024, sk, 0);
		__syncwarp();
		if (c >= 0)
			for (int d = lane; d < 256; d += 32) kcache[size_t(c) * 256 + d] = kr[d];
	} else {
		for (int d = lane; d < 256; d += 32) {
			float val;
			if (nsplit > 0) {
				val = raw(1280 + d, sv, d);
				v[size_t(s) * 256 + d] = val;
			} else {
				val = v[size_t(s) * 256 + d];
			}
			if (c >= 0) vcache[size_t(c) * 256 + d] = val;
		}
	}
}

// ops::attention_prefill, reference ops.hpp:377-526: causal; on sliding-window
// layers query s sees keys max(0, s - window) .. s (window + 1 keys, :437-443).
// q,o [S][4][256], k,v [S][256] (the prompt's own activations, not the cache).
// One CTA = 8 consecutive queries, one warp per query handling the 4 heads that
// share the KV head. The CTA walks the union of its queries' key ranges in
// tiles of 16 keys staged in shared memory (K and V, 32 KiB); the next tile is
// fetched into registers while the current one is consumed, so the L2 latency of
// a key row is paid once per tile instead of once per key.
constexpr int AP_QPB = 8;     // queries per CTA
constexpr int AP_TILE = 16;   // keys per shared-memory tile
constexpr int AP_BLK_SMEM = 4 * AP_TILE * 256 * 4;  // attn_prefill_blk_kernel: two K and two V tiles (dynamic shared memory)

__global__ void __launch_bounds__(256) attn_prefill_kernel(float *o, const float *q, const float *k, const float *v, int S,
                                                           int is_local, int window) {
	{
		const size_t r0 = size_t(blockIdx.y) * S;  // several prompts of the same length share a launch: blockIdx.y is the prompt
		o += r0 * 1024;
		q += r0 * 1024;
		k += r0 * 256;
		v += r0 * 256;
	}
	__shared__ __align__(16) float ks[AP_TILE][256];
	__shared__ __align__(16) float vs[AP_TILE][256];
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int s0 = blockIdx.x * AP_QPB;
	const int s = s0 + warp;              // this warp's query (may be >= S: then it only helps loading)
	const int s_last = min(S - 1, s0 + AP_QPB - 1);
	int cta_j0 = 0;
	if (is_local) cta_j0 = (s0 >= window) ? s0 - window : 0;
	int my_j0 = 0;
	if (is_local) my_j0 = (s >= window) ? s - window : 0;
	float4 q0[4], q1[4], o0[4], o1[4];
	float m[4], l[4];
#pragma unroll
	for (int h = 0; h < 4; h++) {
		if (s < S) {
			const float *qr = q + size_t(s) * 1024 + h * 256;
			q0[h] = *reinterpret_cast<const float4 *>(qr + 4 * lane);
			q1[h] = *reinterpret_cast<const float4 *>(qr + 128 + 4 * lane);
		} else {
			q0[h] = make_float4(0.f, 0.f, 0.f, 0.f);
			q1[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		}
		// the reference multiplies the score by 1/16 after the dot product (ops.hpp:463); scaling q
		// by the same power of two first is exact
		q0[h].x *= 0.0625f; q0[h].y *= 0.0625f; q0[h].z *= 0.0625f; q0[h].w *= 0.0625f;
		q1[h].x *= 0.0625f; q1[h].y *= 0.0625f; q1[h].z *= 0.0625f; q1[h].w *= 0.0625f;
		o0[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		o1[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		m[h] = -INFINITY;
		l[h] = 0.0f;
	}
	// tile loads: 16 rows x 256 floats x {K,V} = 2048 float4; thread t takes float4 slots t, t+256, ... (4 of K, 4 of V)
	float4 pk[4], pv[4];
	auto fetch = [&](int jt) {
#pragma unroll
		for (int u = 0; u < 4; u++) {
			const int slot = tid + 256 * u, r = slot >> 6, c4 = slot & 63;
			const int j = jt + r;
			if (j <= s_last) {
				pk[u] = *reinterpret_cast<const float4 *>(k + size_t(j) * 256 + 4 * c4);
				pv[u] = *reinterpret_cast<const float4 *>(v + size_t(j) * 256 + 4 * c4);
			} else {
				pk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
				pv[u] = pk[u];
			}
		}
	};
	fetch(cta_j0);
	for (int jt = cta_j0; jt <= s_last; jt += AP_TILE) {
		__syncthreads();  // previous tile fully consumed
#pragma unroll
		for (int u = 0; u < 4; u++) {
			const int slot = tid + 256 * u, r = slot >> 6, c4 = slot & 63;
			*reinterpret_cast<float4 *>(&ks[r][4 * c4]) = pk[u];
			*reinterpret_cast<float4 *>(&vs[r][4 * c4]) = pv[u];
		}
		__syncthreads();
		if (jt + AP_TILE <= s_last) fetch(jt + AP_TILE);
		if (s < S) {
			const int ja = max(jt, my_j0), jb = min(jt + AP_TILE - 1, s);
			for (int j = ja; j <= jb; j++) {
				const int r = j - jt;
				const float4 k0v = *reinterpret_cast<const float4 *>(&ks[r][4 * lane]);
				const float4 k1v = *reinterpret_cast<const float4 *>(&ks[r][128 + 4 * lane]);
				const float4 v0v = *reinterpret_cast<const float4 *>(&vs[r][4 * lane]);
				const float4 v1v = *reinterpret_cast<const float4 *>(&vs[r][128 + 4 * lane]);
				float sc[4];
#pragma unroll
				for (int h = 0; h < 4; h++) {
					float t = q0[h].x * k0v.x;
					t = fmaf(q0[h].y, k0v.y, t);
					t = fmaf(q0[h].z, k0v.z, t);
					t = fmaf(q0[h].w, k0v.w, t);
					t = fmaf(q1[h].x, k1v.x, t);
					t = fmaf(q1[h].y, k1v.y, t);
					t = fmaf(q1[h].z, k1v.z, t);
					t = fmaf(q1[h].w, k1v.w, t);
					sc[h] = t;
				}
#pragma unroll
				for (int of = 16; of > 0; of >>= 1) {
#pragma unroll
					for (int h = 0; h < 4; h++) sc[h] += __shfl_xor_sync(0xffffffffu, sc[h], of);
				}
#pragma unroll
				for (int h = 0; h < 4; h++) {
					const float mn = fmaxf(m[h], sc[h]);
					const float corr = expf(m[h] - mn);
					const float p = expf(sc[h] - mn);
					l[h] = fmaf(l[h], corr, p);
					o0[h].x = fmaf(p, v0v.x, o0[h].x * corr);
					o0[h].y = fmaf(p, v0v.y, o0[h].y * corr);
					o0[h].z = fmaf(p, v0v.z, o0[h].z * corr);
					o0[h].w = fmaf(p, v0v.w, o0[h].w * corr);
					o1[h].x = fmaf(p, v1v.x, o1[h].x * corr);
					o1[h].y = fmaf(p, v1v.y, o1[h].y * corr);
					o1[h].z = fmaf(p, v1v.z, o1[h].z * corr);
					o1[h].w = fmaf(p, v1v.w, o1[h].w * corr);
					m[h] = mn;
				}
			}
		}
	}
	if (s >= S) return;
#pragma unroll
	for (int h = 0; h < 4; h++) {
		const float inv = 1.0f / l[h];
		float *orow = o + size_t(s) * 1024 + h * 256;
		*reinterpret_cast<float4 *>(orow + 4 * lane) = make_float4(o0[h].x * inv, o0[h].y * inv, o0[h].z * inv, o0[h].w * inv);
		*reinterpret_cast<float4 *>(orow + 128 + 4 * lane) =
		    make_float4(o1[h].x * inv, o1[h].y * inv, o1[h].z * inv, o1[h].w * inv);
	}
}

// Long prompts (the O(S^2) regime): the same CTA shape as attn_prefill_kernel (8 queries, a warp per
// query with its four heads, 16-key tiles in shared memory), but a warp takes FOUR keys at a time:
//  * the 16 partial dot products of a lane (4 keys x 4 heads) are reduced over the warp with a
//    reduce-scatter butterfly (16 shuffles instead of 80): afterwards lane L holds the finished score
//    of key (L >> 3), head (L >> 1) & 3;
//  * the softmax state (running max, denominator) of a head lives on the lanes that own it; each lane
//    evaluates ONE probability and one rescale factor per block (2 exp instead of 32 per lane), and
//    the 16 probabilities and 4 rescale factors are then broadcast by index shuffles;
//  * the output is rescaled once per block of four keys.
// The running max advances per block instead of per key; the result equals the per-key recurrence of
// the reference (ops.hpp:465-480) up to fp32 rounding.
__global__ void __launch_bounds__(256, 2) attn_prefill_blk_kernel(float *o, const float *q, const float *k, const float *v, int S,
                                                               int is_local, int window) {
	pdl_trigger();
	pdl_wait();
	{
		const size_t r0 = size_t(blockIdx.y) * S;  // several prompts of the same length share a launch: blockIdx.y is the prompt
		o += r0 * 1024;
		q += r0 * 1024;
		k += r0 * 256;
		v += r0 * 256;
	}
	// two K tiles and two V tiles (64 KiB): the next tile is copied asynchronously while this one is consumed
	extern __shared__ __align__(16) float ap_smem[];
	float (*ksb)[AP_TILE][256] = reinterpret_cast<float (*)[AP_TILE][256]>(ap_smem);
	float (*vsb)[AP_TILE][256] = reinterpret_cast<float (*)[AP_TILE][256]>(ap_smem + 2 * AP_TILE * 256);
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int s0 = blockIdx.x * AP_QPB;
	const int s = s0 + warp;              // this warp's query (may be >= S: then it only helps loading)
	const int s_last = min(S - 1, s0 + AP_QPB - 1);
	int cta_j0 = 0;
	if (is_local) cta_j0 = (s0 >= window) ? s0 - window : 0;
	int my_j0 = 0;
	if (is_local) my_j0 = (s >= window) ? s - window : 0;
	// Slot order: a lane keeps its heads and the keys of a block in a lane-dependent order (slot ^ hperm,
	// slot ^ kperm), chosen so that every round of the reduce-scatter below keeps the lower half of the
	// slots and sends the upper half on every lane, without selects.
	const int hperm = (lane >> 1) & 3, kperm = (lane >> 3) & 3;
	float4 q0[4], q1[4], o0[4], o1[4];
#pragma unroll
	for (int h = 0; h < 4; h++) {  // h: head slot; the head is h ^ hperm
		if (s < S) {
			const float *qr = q + size_t(s) * 1024 + (h ^ hperm) * 256;
			q0[h] = *reinterpret_cast<const float4 *>(qr + 4 * lane);
			q1[h] = *reinterpret_cast<const float4 *>(qr + 128 + 4 * lane);
		} else {
			q0[h] = make_float4(0.f, 0.f, 0.f, 0.f);
			q1[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		}
		// 1/16 = 1/sqrt(256): a power of two, exact on q (the reference scales the score, ops.hpp:463)
		q0[h].x *= 0.0625f; q0[h].y *= 0.0625f; q0[h].z *= 0.0625f; q0[h].w *= 0.0625f;
		q1[h].x *= 0.0625f; q1[h].y *= 0.0625f; q1[h].z *= 0.0625f; q1[h].w *= 0.0625f;
		o0[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		o1[h] = make_float4(0.f, 0.f, 0.f, 0.f);
	}
	const int own_kk = lane >> 3;        // key of the block whose score this lane holds after the butterfly
	float m_own = -INFINITY, l_own = 0.0f;  // softmax state of head (lane >> 1) & 3
	// tile copy: 16 rows x 256 floats x {K, V} = 2048 x 16 bytes, 8 per thread; rows past the CTA's last
	// key are zero-filled (source size 0 at a clamped address)
	auto issue = [&](int jt, int buf) {
#pragma unroll
		for (int u = 0; u < 4; u++) {
			const int slot = tid + 256 * u, r = slot >> 6, c4 = slot & 63;
			const int j = jt + r;
			const unsigned nbytes = (j <= s_last) ? 16u : 0u;
			const size_t src = size_t(min(j, s_last)) * 256 + 4 * c4;
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&ksb[buf][r][4 * c4])), "l"(k + src), "r"(nbytes) : "memory");
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&vsb[buf][r][4 * c4])), "l"(v + src), "r"(nbytes) : "memory");
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	issue(cta_j0, 0);
	int buf = 0;
	for (int jt = cta_j0; jt <= s_last; jt += AP_TILE, buf ^= 1) {
		// (every thread has passed the barrier that ends the previous iteration: buffer buf ^ 1 is free)
		if (jt + AP_TILE <= s_last) {
			issue(jt + AP_TILE, buf ^ 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile's copies of this thread are done
		} else {
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		}
		__syncthreads();  // ... and everyone else's
		float (*ks)[256] = ksb[buf];
		float (*vs)[256] = vsb[buf];
		if (s < S) {
#pragma unroll 1
		for (int r0 = 0; r0 < AP_TILE; r0 += 4) {
			const int jb0 = jt + r0;  // first key of the block
			if (jb0 > s || jb0 + 3 < my_j0) continue;  // no key of the block is visible to this query
			// ---- 16 partial scores: x[key slot * 4 + head slot]
			float x[16];
#pragma unroll
			for (int kk = 0; kk < 4; kk++) {
				const float4 k0v = *reinterpret_cast<const float4 *>(&ks[r0 + (kk ^ kperm)][4 * lane]);
				const float4 k1v = *reinterpret_cast<const float4 *>(&ks[r0 + (kk ^ kperm)][128 + 4 * lane]);
#pragma unroll
				for (int h = 0; h < 4; h++) {
					float t = q0[h].x * k0v.x;
					t = fmaf(q0[h].y, k0v.y, t);
					t = fmaf(q0[h].z, k0v.z, t);
					t = fmaf(q0[h].w, k0v.w, t);
					t = fmaf(q1[h].x, k1v.x, t);
					t = fmaf(q1[h].y, k1v.y, t);
					t = fmaf(q1[h].z, k1v.z, t);
					t = fmaf(q1[h].w, k1v.w, t);
					x[kk * 4 + h] = t;
				}
			}
			// ---- reduce-scatter over the warp: every round halves the values a lane carries. The partner of a
			// round differs in exactly the permutation bit that the round splits on, so its upper-half slot
			// holds the same (key, head) as this lane's lower-half slot.
			float y8[8], y4[4], y2[2];
#pragma unroll
			for (int i = 0; i < 8; i++) y8[i] = x[i] + __shfl_xor_sync(0xffffffffu, x[i + 8], 16);
#pragma unroll
			for (int i = 0; i < 4; i++) y4[i] = y8[i] + __shfl_xor_sync(0xffffffffu, y8[i + 4], 8);
#pragma unroll
			for (int i = 0; i < 2; i++) y2[i] = y4[i] + __shfl_xor_sync(0xffffffffu, y4[i + 2], 4);
			float sc = y2[0] + __shfl_xor_sync(0xffffffffu, y2[1], 2);
			sc += __shfl_xor_sync(0xffffffffu, sc, 1);
			// lane L now holds the score of key jb0 + (L >> 3) for head (L >> 1) & 3
			const int j_own = jb0 + own_kk;
			if (j_own > s || j_own < my_j0) sc = -INFINITY;  // outside the causal / sliding window
			// ---- softmax step of the block on the owning lanes
			float mb = fmaxf(sc, __shfl_xor_sync(0xffffffffu, sc, 8));
			mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
			const float mn = fmaxf(m_own, mb);            // finite: at least one key of the block is visible
			const float corr = expf(m_own - mn);          // exp(-inf) = 0 on the first block
			const float pr = expf(sc - mn);               // 0 for a masked key
			float ps = pr + __shfl_xor_sync(0xffffffffu, pr, 8);
			ps += __shfl_xor_sync(0xffffffffu, ps, 16);
			l_own = fmaf(l_own, corr, ps);
			m_own = mn;
			// ---- everyone needs the 4 rescale factors and the 16 probabilities
			float cf[4], pa[16];
#pragma unroll
			for (int h = 0; h < 4; h++) cf[h] = __shfl_sync(0xffffffffu, corr, 2 * (h ^ hperm));
#pragma unroll
			for (int i = 0; i < 16; i++) pa[i] = __shfl_sync(0xffffffffu, pr, 2 * (i ^ hperm));  // [key][head slot]
#pragma unroll
			for (int h = 0; h < 4; h++) {
				o0[h].x *= cf[h]; o0[h].y *= cf[h]; o0[h].z *= cf[h]; o0[h].w *= cf[h];
				o1[h].x *= cf[h]; o1[h].y *= cf[h]; o1[h].z *= cf[h]; o1[h].w *= cf[h];
			}
#pragma unroll
			for (int kk = 0; kk < 4; kk++) {
				const float4 v0v = *reinterpret_cast<const float4 *>(&vs[r0 + kk][4 * lane]);
				const float4 v1v = *reinterpret_cast<const float4 *>(&vs[r0 + kk][128 + 4 * lane]);
#pragma unroll
				for (int h = 0; h < 4; h++) {
					const float pp = pa[kk * 4 + h];
					o0[h].x = fmaf(pp, v0v.x, o0[h].x);
					o0[h].y = fmaf(pp, v0v.y, o0[h].y);
					o0[h].z = fmaf(pp, v0v.z, o0[h].z);
					o0[h].w = fmaf(pp, v0v.w, o0[h].w);
					o1[h].x = fmaf(pp, v1v.x, o1[h].x);
					o1[h].y = fmaf(pp, v1v.y, o1[h].y);
					o1[h].z = fmaf(pp, v1v.z, o1[h].z);
					o1[h].w = fmaf(pp, v1v.w, o1[h].w);
				}
			}
		}
		}
		__syncthreads();  // the tile is consumed: the next iteration may overwrite the other buffer's partner
	}
	if (s >= S) return;
#pragma unroll
	for (int h = 0; h < 4; h++) {
		const float inv = 1.0f / __shfl_sync(0xffffffffu, l_own, 2 * (h ^ hperm));
		float *orow = o + size_t(s) * 1024 + (h ^ hperm) * 256;
		*reinterpret_cast<float4 *>(orow + 4 * lane) = make_float4(o0[h].x * inv, o0[h].y * inv, o0[h].z * inv, o0[h].w * inv);
		*reinterpret_cast<float4 *>(orow + 128 + 4 * lane) =
		    make_float4(o1[h].x * inv, o1[h].y * inv, o1[h].z * inv, o1[h].w * inv);
	}
}

// Short prompts: with one query per warp the kernels above run on only S/8 CTAs, and a (query, head)'s walk
// over its keys is a chain of dependent shuffles and exponentials that one warp cannot hide. Here a CTA of
// 32 warps takes two queries; a warp owns one (query, head) and ONE of the four 4-key blocks of every
// 16-key tile (the keys of a (query, head) are split four ways). Per block, as in attn_prefill_blk_kernel:
// the four partial scores of a lane are reduce-scattered over the warp, the running max advances once,
// every lane evaluates one probability, and the four probabilities are broadcast. The four partial
// results (max, sum, output) of a (query, head) are merged through shared memory at the end.
constexpr int APS_THREADS = 1024;
__global__ void __launch_bounds__(APS_THREADS, 1) attn_prefill_small_kernel(float *o, const float *q, const float *k, const float *v,
                                                                           int S, int is_local, int window) {
	pdl_trigger();
	pdl_wait();
	{
		const size_t r0 = size_t(blockIdx.y) * S;  // several prompts of the same length share a launch: blockIdx.y is the prompt
		o += r0 * 1024;
		q += r0 * 1024;
		k += r0 * 256;
		v += r0 * 256;
	}
	__shared__ __align__(16) float kv[2][AP_TILE][256];  // K tile, V tile; afterwards the 32 warps' partial outputs
	__shared__ float ml[32][2];
	float (*ks)[256] = kv[0];
	float (*vs)[256] = kv[1];
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int s0 = blockIdx.x * 2;
	const int part = warp & 3, h = (warp >> 2) & 3;  // this warp's 4-key block of every tile, and its head
	const int s = s0 + (warp >> 4);                  // its query (may be >= S: then the warp only helps loading)
	const int s_last = min(S - 1, s0 + 1);
	int cta_j0 = 0;
	if (is_local) cta_j0 = (s0 >= window) ? s0 - window : 0;
	int my_j0 = 0;
	if (is_local) my_j0 = (s >= window) ? s - window : 0;
	float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0, o0 = q0, o1 = q0;
	float m = -INFINITY, l = 0.0f;
	if (s < S) {
		const float *qr = q + size_t(s) * 1024 + h * 256;
		q0 = *reinterpret_cast<const float4 *>(qr + 4 * lane);
		q1 = *reinterpret_cast<const float4 *>(qr + 128 + 4 * lane);
		q0.x *= 0.0625f; q0.y *= 0.0625f; q0.z *= 0.0625f; q0.w *= 0.0625f;  // exact: see attn_prefill_kernel
		q1.x *= 0.0625f; q1.y *= 0.0625f; q1.z *= 0.0625f; q1.w *= 0.0625f;
	}
	// one float4 of K and one of V per thread and tile, fetched a tile ahead
	const int fr = tid >> 6, fc4 = tid & 63;
	float4 pk, pv;
	auto fetch = [&](int jt) {
		const int j = jt + fr;
		if (j <= s_last) {
			pk = *reinterpret_cast<const float4 *>(k + size_t(j) * 256 + 4 * fc4);
			pv = *reinterpret_cast<const float4 *>(v + size_t(j) * 256 + 4 * fc4);
		} else {
			pk = make_float4(0.f, 0.f, 0.f, 0.f);
			pv = pk;
		}
	};
	fetch(cta_j0);
	for (int jt = cta_j0; jt <= s_last; jt += AP_TILE) {
		__syncthreads();  // previous tile fully consumed
		*reinterpret_cast<float4 *>(&ks[fr][4 * fc4]) = pk;
		*reinterpret_cast<float4 *>(&vs[fr][4 * fc4]) = pv;
		__syncthreads();
		if (jt + AP_TILE <= s_last) fetch(jt + AP_TILE);
		// this warp's block: keys j4 .. j4 + 3, of which [lo, hi] are visible to its query
		const int j4 = jt + 4 * part;
		const int lo = max(j4, my_j0), hi = min(j4 + 3, s);
		if (s < S && lo <= hi) {
			float sc[4];
#pragma unroll
			for (int u = 0; u < 4; u++) {
				const int r = 4 * part + u;  // (rows outside [lo, hi] hold other keys or zeros; their scores are not used)
				const float4 k0v = *reinterpret_cast<const float4 *>(&ks[r][4 * lane]);
				const float4 k1v = *reinterpret_cast<const float4 *>(&ks[r][128 + 4 * lane]);
				float t = q0.x * k0v.x;
				t = fmaf(q0.y, k0v.y, t);
				t = fmaf(q0.z, k0v.z, t);
				t = fmaf(q0.w, k0v.w, t);
				t = fmaf(q1.x, k1v.x, t);
				t = fmaf(q1.y, k1v.y, t);
				t = fmaf(q1.z, k1v.z, t);
				t = fmaf(q1.w, k1v.w, t);
				sc[u] = t;
			}
			// reduce-scatter over the warp (6 shuffles instead of 20): afterwards lane L holds the finished
			// score of key j4 + (L >> 3)
			float z;
			{
				const bool up = lane & 16, up8 = lane & 8;
				const float y0 = (up ? sc[2] : sc[0]) + __shfl_xor_sync(0xffffffffu, up ? sc[0] : sc[2], 16);
				const float y1 = (up ? sc[3] : sc[1]) + __shfl_xor_sync(0xffffffffu, up ? sc[1] : sc[3], 16);
				z = (up8 ? y1 : y0) + __shfl_xor_sync(0xffffffffu, up8 ? y0 : y1, 8);
			}
			z += __shfl_xor_sync(0xffffffffu, z, 4);
			z += __shfl_xor_sync(0xffffffffu, z, 2);
			z += __shfl_xor_sync(0xffffffffu, z, 1);
			const int jmine = j4 + (lane >> 3);
			if (jmine < lo || jmine > hi) z = -INFINITY;  // outside this query's window or past its last key
			// one softmax step for the block of four keys
			float mb = fmaxf(z, __shfl_xor_sync(0xffffffffu, z, 8));
			mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
			const float mn = fmaxf(m, mb);      // finite: the block has a visible key
			const float corr = expf(m - mn);    // exp(-inf) = 0 on this warp's first block
			const float pr = expf(z - mn);      // this lane's key; 0 when masked
			float pb[4];
#pragma unroll
			for (int u = 0; u < 4; u++) pb[u] = __shfl_sync(0xffffffffu, pr, 8 * u);
			l = fmaf(l, corr, (pb[0] + pb[1]) + (pb[2] + pb[3]));
			m = mn;
			o0.x *= corr; o0.y *= corr; o0.z *= corr; o0.w *= corr;
			o1.x *= corr; o1.y *= corr; o1.z *= corr; o1.w *= corr;
#pragma unroll
			for (int u = 0; u < 4; u++) {
				const int r = 4 * part + u;  // (masked keys: p is 0, the row holds finite values)
				const float4 v0v = *reinterpret_cast<const float4 *>(&vs[r][4 * lane]);
				const float4 v1v = *reinterpret_cast<const float4 *>(&vs[r][128 + 4 * lane]);
				o0.x = fmaf(pb[u], v0v.x, o0.x);
				o0.y = fmaf(pb[u], v0v.y, o0.y);
				o0.z = fmaf(pb[u], v0v.z, o0.z);
				o0.w = fmaf(pb[u], v0v.w, o0.w);
				o1.x = fmaf(pb[u], v1v.x, o1.x);
				o1.y = fmaf(pb[u], v1v.y, o1.y);
				o1.z = fmaf(pb[u], v1v.z, o1.z);
				o1.w = fmaf(pb[u], v1v.w, o1.w);
			}
		}
	}
	// merge the four partial results of every (query, head): partial outputs over the K / V tiles
	__syncthreads();
	float *po = &kv[0][0][0];  // [32 warps][256]
	*reinterpret_cast<float4 *>(po + warp * 256 + 4 * lane) = o0;
	*reinterpret_cast<float4 *>(po + warp * 256 + 128 + 4 * lane) = o1;
	if (lane == 0) {
		ml[warp][0] = m;
		ml[warp][1] = l;
	}
	__syncthreads();
	// 8 (query, head) pairs x 256 values over 1024 threads: two values per thread
#pragma unroll
	for (int rep = 0; rep < 2; rep++) {
		const int idx = tid + rep * APS_THREADS;
		const int pair = idx >> 8, d = idx & 255;  // pair = warp >> 2 of the four warps that share it
		const int sq = s0 + (pair >> 2);
		if (sq >= S) continue;
		float mm = -INFINITY;
#pragma unroll
		for (int t = 0; t < 4; t++) mm = fmaxf(mm, ml[4 * pair + t][0]);  // finite: a query sees itself
		float den = 0.0f, num = 0.0f;
#pragma unroll
		for (int t = 0; t < 4; t++) {
			const float wgt = expf(ml[4 * pair + t][0] - mm);  // 0 for a part without visible keys (max -inf, sum 0)
			den = fmaf(ml[4 * pair + t][1], wgt, den);
			num = fmaf(po[(4 * pair + t) * 256 + d], wgt, num);
		}
		o[size_t(sq) * 1024 + (pair & 3) * 256 + d] = num / den;
	}
}

}  // namespace tg
