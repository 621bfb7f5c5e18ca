// Decode-step kernels (one token per sequence): embedding, the int8
// weight-only matvec with fused norm prologues / GeGLU epilogue, and split-KV
// attention over the cache. All are HBM-bandwidth bound; none uses tensor cores.
#pragma once
#include <cooperative_groups.h>

#include "tg_common.cuh"

namespace tg {

// =========================================================== embedding
// ops::embedding_decode, reference ops.hpp:574-616:
//   h[d] = scale[d] * (sqrt(D) * float(wte[tok, d]))
// One CTA per sequence. Also latches the position this step works at:
// step_pos = next_pos, next_pos += 1 (KVCache::position_ptr, decode.hpp:69).
struct EmbedArgs {
	const int8_t *wte;
	const float *scales;
	const int *tok;   // [B]
	float *h;         // [B][D]
	int *step_pos;    // [B]
	int *next_pos;    // [B]
	int *err_flag;    // set to 1 if a token id is out of range
	int D, V;
	float sqrtD;
};

__global__ void embed_decode_kernel(EmbedArgs a) {
	pdl_trigger();
	pdl_wait();
	int b = blockIdx.x;
	int tok = a.tok[b];
	if (tok < 0 || tok >= a.V) {
		if (threadIdx.x == 0) *a.err_flag = 1;
		tok = 0;
	}
	const int8_t *row = a.wte + size_t(tok) * a.D;
	for (int d = threadIdx.x; d < a.D; d += blockDim.x) a.h[size_t(b) * a.D + d] = a.scales[d] * (a.sqrtD * float(row[d]));
	if (threadIdx.x == 0) {
		int p = a.next_pos[b];
		a.step_pos[b] = p;
		a.next_pos[b] = p + 1;
	}
}

// =========================================================== int8 matvec
// y[n] = scale[n] * sum_k x[k] * W[k,n]   (gemv::qgemv, reference linalg.hpp:41-108)
//
// W is [K,N] row-major int8 exactly as in gemma_i8.bin, so consecutive columns
// are consecutive bytes: a lane owns 16 columns (one 128-bit load per row), 8
// lanes cover a 128-column tile and the 4 lane groups of a warp take 4
// different rows, so one warp-wide load instruction fetches four full 128-byte
// lines. A CTA (8 warps) walks 32 rows per iteration over its K-chunk.
//
// Small-N matrices are split along K across CTAs (grid.y); partial sums go to
// a scratch array and the last CTA to finish a column tile (ticket counter)
// adds them in split order — deterministic, no floating-point atomics.
//
// Prologues build the CTA's slice of x in shared memory:
//   PRO_PLAIN    x = in
//   PRO_NORM     x = rmsnorm(h; w_pre)
//   PRO_RESNORM  h' = h + rmsnorm(t; w_post);  x = rmsnorm(h'; w_pre)   (CTA 0,0 stores h')
//   (modules::attention / modules::mlp sandwich norms, reference modules.hpp:140,166-168,209,218-219)
// Epilogues (by the finishing CTA of a tile):
//   EPI_SCALE    out = scale * sum
//   EPI_GEGLU    two matrices (up, gate) share the tile: out = lut(sg*gate) * (su*up)
//   (ops::gelu + ops::mul, reference modules.hpp:213-215)
constexpr int MV_TN = 128;
constexpr int MV_THREADS = 256;
constexpr int MV_NWARPS = MV_THREADS / 32;
constexpr int MV_ROWS_PER_ITER = 32;

enum { PRO_PLAIN = 0, PRO_NORM = 1, PRO_RESNORM = 2 };
enum { EPI_SCALE = 0, EPI_GEGLU = 1 };

struct MvSeg {
	const int8_t *w;
	const float *scale;
	int N;        // row stride of this matrix
	int out_off;  // column offset of this segment in the output row
	int tile0;    // first tile index of this segment
};

struct MvArgs {
	MvSeg seg[3];
	int nseg;
	int ntiles;      // total column tiles over all segments (EPI_GEGLU: tiles of one matrix)
	int K;           // rows
	int kc;          // rows per K-split (multiple of 32)
	int nsplit;      // == gridDim.y
	int B;           // sequences in this launch (<= MB)
	int part_stride; // columns per (split, b) row of the partial buffer
	int out_stride;  // floats per output row
	// prologue inputs
	const float *x;       // PRO_PLAIN: [B][K]
	const float *h;       // PRO_NORM / PRO_RESNORM: residual stream [B][K]
	const float *t;       // PRO_RESNORM: branch output to be post-normed [B][K]
	const float *w_post;  // [K]
	const float *w_pre;   // [K]
	float *h_out;         // PRO_RESNORM: updated residual stream [B][K] (must differ from h)
	float *x_out;         // optional copy of the normed input (parity read-back), may be null
	// split-K machinery
	float *partial;       // [nsplit][B][part_stride]
	unsigned *tickets;    // [ntiles], zero on entry, zero on exit
	float *out;           // [B][out_stride]
	GeluLut lut;          // EPI_GEGLU
};

template <int MB>
__device__ __forceinline__ void mv_accumulate(float (&acc)[MB][16], const int4 &v, const float (&xv)[MB]) {
	const uint32_t words[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
#pragma unroll
	for (int j = 0; j < 4; j++) {
		float f[4];
		i8x4_to_f32(words[j], f);
#pragma unroll
		for (int b = 0; b < MB; b++) {
#pragma unroll
			for (int i = 0; i < 4; i++) acc[b][4 * j + i] = fmaf(xv[b], f[i], acc[b][4 * j + i]);
		}
	}
}

// Walks rows [k0, k0+kc) of one 128-column tile; returns per-thread sums for
// its 16 columns over the rows this thread visited.
template <int MB>
__device__ __forceinline__ void mv_tile_rows(float (&acc)[MB][16], const int8_t *wcol, int N, int kc, const float *xs,
                                             int xs_stride) {
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int sub = lane >> 3;
	const int r0 = warp * 4 + sub;  // row within a 32-row iteration
	const int8_t *p = wcol + size_t(r0) * N;
	const size_t step = size_t(MV_ROWS_PER_ITER) * N;
	const int iters = kc / MV_ROWS_PER_ITER;
	int it = 0;
	// eight 16-byte loads in flight per thread (32 KB per CTA): a K-split slice of 256 rows is one round trip to DRAM
	for (; it + 8 <= iters; it += 8) {
		int4 v[8];
#pragma unroll
		for (int u = 0; u < 8; u++) v[u] = ld_stream_int4(p + u * step);
		p += 8 * step;
		const int r = it * MV_ROWS_PER_ITER + r0;
#pragma unroll
		for (int u = 0; u < 8; u++) {
			float xv[MB];
#pragma unroll
			for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r + 32 * u];
			mv_accumulate<MB>(acc, v[u], xv);
		}
	}
	for (; it + 4 <= iters; it += 4) {
		int4 v0 = ld_stream_int4(p);
		int4 v1 = ld_stream_int4(p + step);
		int4 v2 = ld_stream_int4(p + 2 * step);
		int4 v3 = ld_stream_int4(p + 3 * step);
		p += 4 * step;
		float xv[MB];
		const int r = it * MV_ROWS_PER_ITER + r0;
#pragma unroll
		for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r];
		mv_accumulate<MB>(acc, v0, xv);
#pragma unroll
		for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r + 32];
		mv_accumulate<MB>(acc, v1, xv);
#pragma unroll
		for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r + 64];
		mv_accumulate<MB>(acc, v2, xv);
#pragma unroll
		for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r + 96];
		mv_accumulate<MB>(acc, v3, xv);
	}
	for (; it < iters; it++) {
		int4 v0 = ld_stream_int4(p);
		p += step;
		float xv[MB];
		const int r = it * MV_ROWS_PER_ITER + r0;
#pragma unroll
		for (int b = 0; b < MB; b++) xv[b] = xs[b * xs_stride + r];
		mv_accumulate<MB>(acc, v0, xv);
	}
}

// Reduce the per-thread sums of one tile across the CTA: over the 4 row groups
// of each warp by shuffle, then over the 8 warps through shared memory.
// On return threads 0..127 hold, for each b, the tile's column (threadIdx.x).
template <int MB>
__device__ __forceinline__ void mv_reduce_cta(float (&acc)[MB][16], float *red /*[MB][NWARPS][128]*/, float (&col)[MB]) {
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
	for (int b = 0; b < MB; b++)
#pragma unroll
		for (int i = 0; i < 16; i++) {
			float v = acc[b][i];
			v += __shfl_xor_sync(0xffffffffu, v, 8);
			v += __shfl_xor_sync(0xffffffffu, v, 16);
			acc[b][i] = v;
		}
	__syncthreads();
	if (lane < 8) {
#pragma unroll
		for (int b = 0; b < MB; b++)
#pragma unroll
			for (int i = 0; i < 16; i++) red[(b * MV_NWARPS + warp) * MV_TN + lane * 16 + i] = acc[b][i];
	}
	__syncthreads();
	if (threadIdx.x < MV_TN) {
#pragma unroll
		for (int b = 0; b < MB; b++) {
			float s = 0.0f;
#pragma unroll
			for (int w = 0; w < MV_NWARPS; w++) s += red[(b * MV_NWARPS + w) * MV_TN + threadIdx.x];
			col[b] = s;
		}
	}
}

template <int MB, int PRO, int EPI>
__global__ void __launch_bounds__(MV_THREADS) qmatvec_kernel(MvArgs a) {
	extern __shared__ float smem[];
	// layout: xs[MB][kc] | hs[MB][K] (norm prologues only) | red[MB][8][128] (x2 for GEGLU) | misc
	float *xs = smem;
	float *hs = xs + MB * a.kc;
	float *red = hs + ((PRO == PRO_PLAIN) ? 0 : MB * a.K);
	float *red2 = red + MB * MV_NWARPS * MV_TN;
	__shared__ float bred[MV_NWARPS];
	__shared__ int s_last;

	const int split = blockIdx.y;
	const int k0 = split * a.kc;
	const int tid = threadIdx.x;

	// ------------------------------------------------------------ prologue
	if (PRO == PRO_PLAIN) {
		for (int b = 0; b < a.B; b++)
			for (int k = tid; k < a.kc; k += MV_THREADS) xs[b * a.kc + k] = a.x[size_t(b) * a.K + k0 + k];
	} else {
		const int D = a.K;
		for (int b = 0; b < a.B; b++) {
			float *hb = hs + b * D;
			if (PRO == PRO_RESNORM) {
				float ss = 0.0f;
				for (int d = tid; d < D; d += MV_THREADS) {
					float v = a.t[size_t(b) * D + d];
					ss = fmaf(v, v, ss);
				}
				ss = block_sum<MV_NWARPS>(ss, bred);
				const float r1 = inv_rms(ss, D);
				for (int d = tid; d < D; d += MV_THREADS) {
					float v = a.t[size_t(b) * D + d];
					hb[d] = a.h[size_t(b) * D + d] + (v * r1) * (a.w_post[d] + 1.0f);
				}
			} else {
				for (int d = tid; d < D; d += MV_THREADS) hb[d] = a.h[size_t(b) * D + d];
			}
			float ss2 = 0.0f;
			for (int d = tid; d < D; d += MV_THREADS) {
				float v = hb[d];
				ss2 = fmaf(v, v, ss2);
			}
			ss2 = block_sum<MV_NWARPS>(ss2, bred);
			const float r2 = inv_rms(ss2, D);
			for (int k = tid; k < a.kc; k += MV_THREADS) xs[b * a.kc + k] = (hb[k0 + k] * r2) * (a.w_pre[k0 + k] + 1.0f);
			if (blockIdx.x == 0 && blockIdx.y == 0) {
				if (PRO == PRO_RESNORM)
					for (int d = tid; d < D; d += MV_THREADS) a.h_out[size_t(b) * D + d] = hb[d];
				if (a.x_out)
					for (int d = tid; d < D; d += MV_THREADS) a.x_out[size_t(b) * D + d] = (hb[d] * r2) * (a.w_pre[d] + 1.0f);
			}
		}
	}
	for (int b = a.B; b < MB; b++)
		for (int k = tid; k < a.kc; k += MV_THREADS) xs[b * a.kc + k] = 0.0f;
	__syncthreads();

	const int lane = tid & 31;
	const int cg = lane & 7;  // 16-column group inside the tile

	// ------------------------------------------------------------ tiles
	for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x) {
		// locate the segment of this tile
		int sidx = 0;
		if (EPI != EPI_GEGLU) {
			while (sidx + 1 < a.nseg && tile >= a.seg[sidx + 1].tile0) sidx++;
		}
		const MvSeg &sg = a.seg[sidx];
		const int n0 = (tile - sg.tile0) * MV_TN;  // first column of the tile inside its matrix

		float acc[MB][16];
#pragma unroll
		for (int b = 0; b < MB; b++)
#pragma unroll
			for (int i = 0; i < 16; i++) acc[b][i] = 0.0f;
		mv_tile_rows<MB>(acc, sg.w + size_t(k0) * sg.N + n0 + cg * 16, sg.N, a.kc, xs, a.kc);
		float col[MB];
		mv_reduce_cta<MB>(acc, red, col);

		float col2[MB];
		if (EPI == EPI_GEGLU) {
			const MvSeg &gg = a.seg[1];
#pragma unroll
			for (int b = 0; b < MB; b++)
#pragma unroll
				for (int i = 0; i < 16; i++) acc[b][i] = 0.0f;
			mv_tile_rows<MB>(acc, gg.w + size_t(k0) * gg.N + n0 + cg * 16, gg.N, a.kc, xs, a.kc);
			mv_reduce_cta<MB>(acc, red2, col2);
		}

		const int pcol = sg.out_off + n0 + tid;  // column in the partial / plain output row
		if (a.nsplit == 1) {
			if (tid < MV_TN) {
				for (int b = 0; b < a.B; b++) {
					if (EPI == EPI_SCALE) {
						a.out[size_t(b) * a.out_stride + pcol] = col[b] * sg.scale[n0 + tid];
					} else {
						float up = col[b] * sg.scale[n0 + tid];
						float gate = col2[b] * a.seg[1].scale[n0 + tid];
						a.out[size_t(b) * a.out_stride + n0 + tid] = a.lut(gate) * up;
					}
				}
			}
			continue;
		}

		// split-K: publish partials, take a ticket, last CTA of the tile finishes
		if (tid < MV_TN) {
			for (int b = 0; b < a.B; b++) {
				float *prow = a.partial + (size_t(split) * a.B + b) * a.part_stride;
				if (EPI == EPI_SCALE) {
					__stcg(prow + pcol, col[b]);
				} else {
					__stcg(prow + n0 + tid, col[b]);
					__stcg(prow + a.seg[1].out_off + n0 + tid, col2[b]);
				}
			}
		}
		__threadfence();
		__syncthreads();
		if (tid == 0) {
			unsigned tk = atomicAdd(&a.tickets[tile], 1u);
			s_last = (tk == unsigned(a.nsplit - 1));
		}
		__syncthreads();
		if (s_last) {
			__threadfence();
			if (tid < MV_TN) {
				for (int b = 0; b < a.B; b++) {
					// the splits are added in ascending order, eight loads in flight at a time (a chain of
					// dependent loads over 30 splits cost more than the matvec itself)
					float s1 = 0.0f, s2 = 0.0f;
					const float *prow0 = a.partial + size_t(b) * a.part_stride;
					const size_t sstride = size_t(a.B) * a.part_stride;
					if (EPI == EPI_SCALE) {
						s1 = sum_splits<true>(prow0 + pcol, sstride, a.nsplit);
					} else {
						s1 = sum_splits<true>(prow0 + n0 + tid, sstride, a.nsplit);
						s2 = sum_splits<true>(prow0 + a.seg[1].out_off + n0 + tid, sstride, a.nsplit);
					}
					if (EPI == EPI_SCALE) {
						a.out[size_t(b) * a.out_stride + pcol] = s1 * sg.scale[n0 + tid];
					} else {
						float up = s1 * sg.scale[n0 + tid];
						float gate = s2 * a.seg[1].scale[n0 + tid];
						a.out[size_t(b) * a.out_stride + n0 + tid] = a.lut(gate) * up;
					}
				}
			}
			if (tid == 0) a.tickets[tile] = 0u;
		}
		__syncthreads();
	}
}

// =========================================================== single-wave matvec (one sequence)
// y[n] = scale[n] * sum_k x[k] W[k,n] for matrices small enough that one wave of CTAs holds all of W in
// flight at once (the layer matrices: 0.6 - 8 MB). Such a launch is bound by its chain of dependent memory
// round trips, so there is exactly one: every CTA requests its whole K-slice of a column tile (and its
// x values) before it waits for anything. K is split over the CTAs of a thread-block cluster
// (gridDim.y = cluster size <= 8) whose partial sums meet in the shared memory of the cluster's first CTA
// (distributed shared memory), added in rank order: no partial-sum buffer, no tickets, no second launch,
// the same bits on every run.
// A column tile is 16 * TPR columns (TPR = 1, 2, 4 threads per row, 16 int8 each); thread t takes columns
// 16 * (t % TPR) .. of rows t / TPR, t / TPR + threads / TPR, ...; at most MVC_MAX_IT rows per thread
// (512 or 256 threads per CTA).
constexpr int MVC_MAX_IT = 10;
constexpr int MVC_MAX_CLUSTER = 8;

template <int TPR, int MVC_THREADS>
__global__ void __launch_bounds__(MVC_THREADS, 1) qmatvec_cluster_kernel(float *y, const float *x, const int8_t *w, const float *scales,
                                                                         int K, int N, int kc) {
	namespace cg = cooperative_groups;
	constexpr int TN = 16 * TPR, ROWS = MVC_THREADS / TPR, MVC_NWARPS = MVC_THREADS / 32;
	cg::cluster_group cluster = cg::this_cluster();
	__shared__ __align__(16) float red[MVC_NWARPS][TN];
	__shared__ float part[MVC_MAX_CLUSTER][TN];  // (used in the cluster's first CTA)
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int n0 = blockIdx.x * TN;
	const int rank = int(cluster.block_rank()), nranks = int(cluster.num_blocks());
	const int k0 = rank * kc;
	const int r0 = tid / TPR, cgp = tid % TPR;
	const int8_t *p = w + size_t(k0 + r0) * N + n0 + cgp * 16;
	int4 v[MVC_MAX_IT];
	float xv[MVC_MAX_IT];
#pragma unroll
	for (int it = 0; it < MVC_MAX_IT; it++) {
		const int r = r0 + it * ROWS;
		v[it] = make_int4(0, 0, 0, 0);
		xv[it] = 0.0f;
		if (r < kc) {
			v[it] = ld_stream_int4(p + size_t(it) * ROWS * N);
			xv[it] = __ldg(x + k0 + r);
		}
	}
	float sc = 0.0f;
	if (rank == 0 && tid < TN) sc = __ldg(scales + n0 + tid);
	float acc[16];
#pragma unroll
	for (int i = 0; i < 16; i++) acc[i] = 0.0f;
#pragma unroll
	for (int it = 0; it < MVC_MAX_IT; it++) {
		const uint32_t words[4] = {uint32_t(v[it].x), uint32_t(v[it].y), uint32_t(v[it].z), uint32_t(v[it].w)};
#pragma unroll
		for (int j = 0; j < 4; j++) {
			float f[4];
			i8x4_to_f32(words[j], f);
#pragma unroll
			for (int i = 0; i < 4; i++) acc[4 * j + i] = fmaf(xv[it], f[i], acc[4 * j + i]);
		}
	}
	// over the rows of a warp (lanes with the same column group), then over the warps
#pragma unroll
	for (int i = 0; i < 16; i++) {
		float s = acc[i];
#pragma unroll
		for (int o = TPR; o < 32; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
		acc[i] = s;
	}
	if (lane < TPR) {
#pragma unroll
		for (int i = 0; i < 16; i += 4)
			*reinterpret_cast<float4 *>(&red[warp][lane * 16 + i]) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
	}
	__syncthreads();
	if (tid < TN) {
		float s = 0.0f;
#pragma unroll
		for (int wi = 0; wi < MVC_NWARPS; wi++) s += red[wi][tid];
		float *dst = cluster.map_shared_rank(&part[rank][tid], 0);  // this rank's row in the first CTA's array
		*dst = s;
	}
	cluster.sync();  // (every thread of every CTA: the stores above are visible to the first CTA behind it)
	if (rank == 0 && tid < TN) {
		float s = 0.0f;
		for (int r = 0; r < nranks; r++) s += part[r][tid];
		y[n0 + tid] = s * sc;
	}
}

// =========================================================== final hidden state
// x = rmsnorm(h + rmsnorm(t; w_post); w_final) per sequence — the prologue of
// the lm_head (reference modules.hpp:242-246) as a kernel of its own, for callers
// that score the vocabulary elsewhere (vocab-sharded lm_head). One CTA per sequence.
__global__ void __launch_bounds__(256) final_hidden_kernel(float *x_out, const float *h, const float *t, const float *w_post,
                                                           const float *w_final, int D) {
	__shared__ float bred[8];
	extern __shared__ float hs[];
	const int b = blockIdx.x, tid = threadIdx.x;
	float ss = 0.0f;
	for (int d = tid; d < D; d += 256) {
		float v = t[size_t(b) * D + d];
		ss = fmaf(v, v, ss);
	}
	ss = block_sum<8>(ss, bred);
	const float r1 = inv_rms(ss, D);
	float ss2 = 0.0f;
	for (int d = tid; d < D; d += 256) {
		float v = h[size_t(b) * D + d] + (t[size_t(b) * D + d] * r1) * (w_post[d] + 1.0f);
		hs[d] = v;
		ss2 = fmaf(v, v, ss2);
	}
	ss2 = block_sum<8>(ss2, bred);
	const float r2 = inv_rms(ss2, D);
	for (int d = tid; d < D; d += 256) x_out[size_t(b) * D + d] = (hs[d] * r2) * (w_final[d] + 1.0f);
}

// =========================================================== attention (decode)
// Per sequence and layer: q/k RMSNorm (per head), RoPE at the token's position,
// KV append into the (ring) cache, then one query against every valid cache
// slot for the 4 query heads that share the single KV head.
// (modules::attention decode branch, reference modules.hpp:151-159;
//  RoPE decode.hpp:136-211; KVCache::update_single decode.hpp:49-70;
//  ops::attention_decode ops.hpp:224-370.)
//
// Grid (nsplit, B). Each CTA repeats the tiny q/k prologue, takes a contiguous
// chunk of cache slots, and writes an un-normalised partial (m, l, o). The last
// CTA of a sequence merges the partials in split order. The softmax is the
// usual running-max form; the reference renormalises its output at every key,
// which is the same function up to rounding.
constexpr int AT_THREADS = 256;
constexpr int AT_NWARPS = 8;
constexpr int AT_HD = 256;
constexpr int AT_NH = 4;

struct AttnArgs {
	const float *qkv;   // [B][1536] = q(4x256) | k(256) | v(256)
	// qkv_nsplit > 0: qkv instead holds the raw K-split partial sums of the grouped q|k|v GEMM,
	// [qkv_nsplit][B][1536], and sq / sk / sv are the column scales (splits are added in ascending order)
	int qkv_nsplit, qkv_B;
	const float *sq, *sk, *sv;
	const float *rmsq;  // [256]
	const float *rmsk;  // [256]
	const float *cosT;  // [n_pos][256]
	const float *sinT;
	float *kcache;      // [B][slots][256]
	float *vcache;
	int slots;          // 512 on local layers, max_pos_global on global layers
	int is_local;
	const int *step_pos;   // [B]
	const int *ring_base;  // [B] prompt length if it filled the ring, else 0 (decode.hpp:98-103)
	float *part;        // [B][nsplit][4*256 + 8]
	unsigned *tickets;  // [B]
	float *out;         // [B][1024]
	int nsplit;
	int *err_flag;
};

__device__ __forceinline__ void norm_rope_head(const float *x, const float *w, const float *cosr, const float *sinr,
                                                float scale, float *dst) {
	// one warp; lane owns d = 4*lane..4*lane+3 and the partner 128 + the same
	const int lane = threadIdx.x & 31;
	float lo[4], hi[4];
	float ss = 0.0f;
#pragma unroll
	for (int i = 0; i < 4; i++) {
		lo[i] = x[4 * lane + i];
		hi[i] = x[128 + 4 * lane + i];
		ss = fmaf(lo[i], lo[i], ss);
		ss = fmaf(hi[i], hi[i], ss);
	}
	ss = warp_sum(ss);
	const float r = inv_rms(ss, AT_HD);
#pragma unroll
	for (int i = 0; i < 4; i++) {
		const int d = 4 * lane + i;
		float a = (lo[i] * r) * (w[d] + 1.0f);
		float b = (hi[i] * r) * (w[d + 128] + 1.0f);
		// y = cos*x + rotate_half(x)*sin, rotate_half = [-x_hi, x_lo]
		float ylo = fmaf(-1.0f * b, sinr[d], cosr[d] * a);
		float yhi = fmaf(a, sinr[d + 128], cosr[d + 128] * b);
		dst[d] = ylo * scale;
		dst[d + 128] = yhi * scale;
	}
}

__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(AttnArgs a) {
	pdl_trigger();
	pdl_wait();
	__shared__ __align__(16) float qs[AT_NH][AT_HD];
	__shared__ __align__(16) float ks[AT_HD];
	__shared__ __align__(16) float vs[AT_HD];
	__shared__ float wm[AT_NWARPS][AT_NH], wl[AT_NWARPS][AT_NH];
	__shared__ __align__(16) float wo[AT_NWARPS][AT_NH][AT_HD];
	__shared__ int s_last;

	const int b = blockIdx.y, split = blockIdx.x;
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	int pos = a.step_pos[b];
	int slot, valid;
	if (a.is_local) {
		int rel = pos - a.ring_base[b];
		slot = rel % a.slots;
		valid = min(pos + 1, a.slots);
	} else {
		if (pos >= a.slots) {  // cache full: refuse to write out of bounds
			if (tid == 0) *a.err_flag = 2;
			pos = a.slots - 1;
		}
		slot = pos;
		valid = pos + 1;
	}
	const float *row = a.qkv + size_t(b) * (AT_NH * AT_HD + 2 * AT_HD);
	if (a.qkv_nsplit > 0) {
		__shared__ __align__(16) float rowbuf[AT_NH * AT_HD + 2 * AT_HD];
		constexpr int NQ = AT_NH * AT_HD + 2 * AT_HD;
		// four consecutive columns x up to eight splits are requested together; the splits are added in
		// ascending order (the order of the reduce kernel)
		const size_t sstride = size_t(a.qkv_B) * NQ;
		for (int n = 4 * tid; n < NQ; n += 4 * AT_THREADS) {
			const float *p = a.qkv + size_t(b) * NQ + n;
			float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
			for (int s0 = 0; s0 < a.qkv_nsplit; s0 += 8) {
				float4 v[8];
#pragma unroll
				for (int q = 0; q < 8; q++) {
					v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
					if (s0 + q < a.qkv_nsplit) v[q] = *reinterpret_cast<const float4 *>(p + size_t(s0 + q) * sstride);
				}
#pragma unroll
				for (int q = 0; q < 8; q++) {
					acc.x += v[q].x;
					acc.y += v[q].y;
					acc.z += v[q].z;
					acc.w += v[q].w;
				}
			}
			const float *sc = n < AT_NH * AT_HD ? a.sq + n : (n < AT_NH * AT_HD + AT_HD ? a.sk + (n - AT_NH * AT_HD) : a.sv + (n - AT_NH * AT_HD - AT_HD));
			const float4 s4 = *reinterpret_cast<const float4 *>(sc);
			*reinterpret_cast<float4 *>(&rowbuf[n]) = make_float4(acc.x * s4.x, acc.y * s4.y, acc.z * s4.z, acc.w * s4.w);
		}
		__syncthreads();
		row = rowbuf;
	}
	const float *cosr = a.cosT + size_t(pos) * AT_HD, *sinr = a.sinT + size_t(pos) * AT_HD;
	if (warp < AT_NH) {
		// the reference scales q by 1/sqrt(256) = 2^-4 before the dot products (ops.hpp:262,283)
		norm_rope_head(row + warp * AT_HD, a.rmsq, cosr, sinr, 0.0625f, qs[warp]);
	} else if (warp == AT_NH) {
		norm_rope_head(row + AT_NH * AT_HD, a.rmsk, cosr, sinr, 1.0f, ks);
	} else if (warp == AT_NH + 1) {
		for (int d = lane; d < AT_HD; d += 32) vs[d] = row[AT_NH * AT_HD + AT_HD + d];
	}
	__syncthreads();

	// chunk of slots for this CTA
	const int chunk = (valid + a.nsplit - 1) / a.nsplit;
	const int j0 = split * chunk, j1 = min(valid, j0 + chunk);
	float *kc = a.kcache + size_t(b) * a.slots * AT_HD;
	float *vc = a.vcache + size_t(b) * a.slots * AT_HD;
	if (slot >= j0 && slot < j1) {
		for (int d = tid; d < AT_HD; d += AT_THREADS) {
			kc[size_t(slot) * AT_HD + d] = ks[d];
			vc[size_t(slot) * AT_HD + d] = vs[d];
		}
	}

	// q in registers: lane owns d = 4*lane..+3 and 128+4*lane..+3 of each head
	float4 q0[AT_NH], q1[AT_NH];
#pragma unroll
	for (int h = 0; h < AT_NH; h++) {
		q0[h] = *reinterpret_cast<const float4 *>(&qs[h][4 * lane]);
		q1[h] = *reinterpret_cast<const float4 *>(&qs[h][128 + 4 * lane]);
	}
	float m[AT_NH], l[AT_NH];
	float4 o0[AT_NH], o1[AT_NH];
#pragma unroll
	for (int h = 0; h < AT_NH; h++) {
		m[h] = -INFINITY;
		l[h] = 0.0f;
		o0[h] = make_float4(0.f, 0.f, 0.f, 0.f);
		o1[h] = make_float4(0.f, 0.f, 0.f, 0.f);
	}
	for (int j = j0 + warp; j < j1; j += AT_NWARPS) {
		float4 k0v, k1v, v0v, v1v;
		if (j == slot) {
			k0v = *reinterpret_cast<const float4 *>(&ks[4 * lane]);
			k1v = *reinterpret_cast<const float4 *>(&ks[128 + 4 * lane]);
			v0v = *reinterpret_cast<const float4 *>(&vs[4 * lane]);
			v1v = *reinterpret_cast<const float4 *>(&vs[128 + 4 * lane]);
		} else {
			const float *kr = kc + size_t(j) * AT_HD, *vr = vc + size_t(j) * AT_HD;
			k0v = __ldcg(reinterpret_cast<const float4 *>(kr + 4 * lane));
			k1v = __ldcg(reinterpret_cast<const float4 *>(kr + 128 + 4 * lane));
			v0v = __ldcg(reinterpret_cast<const float4 *>(vr + 4 * lane));
			v1v = __ldcg(reinterpret_cast<const float4 *>(vr + 128 + 4 * lane));
		}
		float s[AT_NH];
#pragma unroll
		for (int h = 0; h < AT_NH; h++) {
			float t = q0[h].x * k0v.x;
			t = fmaf(q0[h].y, k0v.y, t);
			t = fmaf(q0[h].z, k0v.z, t);
			t = fmaf(q0[h].w, k0v.w, t);
			t = fmaf(q1[h].x, k1v.x, t);
			t = fmaf(q1[h].y, k1v.y, t);
			t = fmaf(q1[h].z, k1v.z, t);
			t = fmaf(q1[h].w, k1v.w, t);
			s[h] = t;
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
			for (int h = 0; h < AT_NH; h++) s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);
		}
#pragma unroll
		for (int h = 0; h < AT_NH; h++) {
			float mn = fmaxf(m[h], s[h]);
			float corr = expf(m[h] - mn);  // exp(-inf) = 0 on the first key
			float p = expf(s[h] - mn);
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
#pragma unroll
	for (int h = 0; h < AT_NH; h++) {
		if (lane == 0) {
			wm[warp][h] = m[h];
			wl[warp][h] = l[h];
		}
		*reinterpret_cast<float4 *>(&wo[warp][h][4 * lane]) = o0[h];
		*reinterpret_cast<float4 *>(&wo[warp][h][128 + 4 * lane]) = o1[h];
	}
	__syncthreads();

	// merge the 8 warps -> CTA partial (thread owns 4 of the 1024 outputs)
	float *prow = a.part + (size_t(b) * a.nsplit + split) * (AT_NH * AT_HD + 8);
	for (int e = tid; e < AT_NH * AT_HD; e += AT_THREADS) {
		const int h = e / AT_HD, d = e % AT_HD;
		float M = -INFINITY;
#pragma unroll
		for (int w = 0; w < AT_NWARPS; w++) M = fmaxf(M, wm[w][h]);
		float L = 0.0f, O = 0.0f;
#pragma unroll
		for (int w = 0; w < AT_NWARPS; w++) {
			float sc = (wm[w][h] == -INFINITY) ? 0.0f : expf(wm[w][h] - M);
			L = fmaf(wl[w][h], sc, L);
			O = fmaf(wo[w][h][d], sc, O);
		}
		__stcg(prow + e, O);
		if (d == 0) {
			__stcg(prow + AT_NH * AT_HD + h, M);
			__stcg(prow + AT_NH * AT_HD + 4 + h, L);
		}
	}
	__threadfence();
	__syncthreads();
	if (tid == 0) {
		unsigned tk = atomicAdd(&a.tickets[b], 1u);
		s_last = (tk == unsigned(a.nsplit - 1));
	}
	__syncthreads();
	if (!s_last) return;
	__threadfence();
	const float *pb = a.part + size_t(b) * a.nsplit * (AT_NH * AT_HD + 8);
	for (int e = tid; e < AT_NH * AT_HD; e += AT_THREADS) {
		const int h = e / AT_HD;
		float M = -INFINITY;
		for (int sp = 0; sp < a.nsplit; sp++) M = fmaxf(M, __ldcg(pb + size_t(sp) * (AT_NH * AT_HD + 8) + AT_NH * AT_HD + h));
		float L = 0.0f, O = 0.0f;
		for (int sp = 0; sp < a.nsplit; sp++) {
			const float *pr = pb + size_t(sp) * (AT_NH * AT_HD + 8);
			float ms = __ldcg(pr + AT_NH * AT_HD + h);
			float sc = (ms == -INFINITY) ? 0.0f : expf(ms - M);
			L = fmaf(__ldcg(pr + AT_NH * AT_HD + 4 + h), sc, L);
			O = fmaf(__ldcg(pr + e), sc, O);
		}
		a.out[size_t(b) * (AT_NH * AT_HD) + e] = O / L;
	}
	if (tid == 0) a.tickets[b] = 0u;
}

}  // namespace tg
