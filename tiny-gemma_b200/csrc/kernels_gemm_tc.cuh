// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
//   C[M,N] = scale[n] * sum_k A[m,k] * W[k,n],  A fp32, W int8 [K,N] row-major
// (gemm::qgemmnn, reference linalg.hpp:210-308, which runs a full-K fp32 FMA
// chain per output).
//
// fp32 accuracy on bf16 tensor cores: int8 weights are exact in bf16; an fp32
// activation is split into three bf16 terms x = hi + mid + lo (8 + 8 + 8
// mantissa bits, each residual computed exactly in fp32), and the three
// products are accumulated into the same fp32 TMEM accumulator. Every product
// is exact; only the fp32 accumulation rounds.
//
//   split_pack_kernel   A fp32 [M,K] -> three bf16 operands, already in the
//                       tensor core's shared-memory layout, tile by tile, so
//                       that a GEMM CTA fetches an operand tile with ONE bulk
//                       copy.
//   qgemm_tc_kernel     one CTA = one BN-column tile of W x MT 128-row tiles of A,
//                       <MT, BN> = <2, 128> or <1, 256> (more rows -> grid.y). Warp
//                       roles: warp 0 producer of the A stages (bulk copies),
//                       warp 6 producer of the int8 W tiles (TMA; its own,
//                       deeper ring), warp 1 MMA issuer, warps 2-5 convert
//                       W int8 -> bf16 into the operand layout and run the
//                       epilogue (TMEM -> registers -> shared memory -> x scale
//                       -> C in row-contiguous stores).
//                       Rings over K in blocks of 32. K may be split over
//                       gridDim.z CTAs (raw partial sums, added in split order
//                       and scaled by qgemm_splitk_reduce_kernel): it fills the
//                       GPU when N/128 is small and keeps the accumulation
//                       chains short — the tensor core truncates when it adds
//                       into the fp32 accumulator, so the error grows with the
//                       chain length (2e-5 at K = 6912 unsplit).
//
// Shared-memory operand layouts (no swizzle): 8 x 8 bf16 "core matrices" of 128
// contiguous bytes (8 rows of 16 bytes).
//   A (K-major):  byte offset of (r, k) in a [128][32] tile
//                 = (r/8)*512 + (k/8)*128 + (r%8)*16 + (k%8)*2
//   B (N-major, as W is stored): byte offset of (k, n) in a [32][BN] tile
//                 = (n/8)*512 + (k/8)*128 + (k%8)*16 + (n%8)*2
// i.e. for both: 128 B between the two 8-wide K groups of an MMA (leading
// offset), 512 B between groups of 8 rows / columns (stride offset). Keeping B
// N-major lets a converter thread turn 8 consecutive int8 of a W row (one
// 8-byte load) into one 16-byte row of a core matrix.
//
// All waits are bounded; a wait that runs out sets *err and the CTA drains and
// frees its TMEM before returning.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "kernels_mega.cuh"  // mbarrier / TMA helpers
#include "tg_common.cuh"

namespace tg {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 32;
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 2;  // 8 KiB: one [128][32] bf16 operand tile
// Two tile shapes of one kernel template <MT, BN>: MT 128-row tiles of A x BN columns of W per CTA.
//   <2, 128>  (small M: one CTA covers up to 256 rows, W converted once for both row tiles)
//   <1, 256>  (large M: every fetched A tile is used against 256 columns; the kernel is bound by the
//              L2 -> SM traffic of the three-term A operand, 6 bytes per activation element)
// Both keep MT * BN * 2 = 512 TMEM columns: two accumulators (K halves) per row tile.
template <int MT, int BN> struct TcShape {
	static constexpr int A_BYTES = 3 * MT * TC_TILE_BYTES;   // one K-block of the three A terms
	static constexpr int W_BYTES = TC_BK * BN;               // int8 W tile
	static constexpr int B_BYTES = BN * TC_BK * 2;           // its bf16 operand form
	// two rings: the large A stages, and the small W / B stages whose loads run further ahead so that the
	// int8 -> bf16 conversion of a K-block is finished before its A tiles land
	static constexpr int NA = (MT == 2) ? 3 : 5;
	static constexpr int NB = 4;
	static constexpr int SMEM = NA * A_BYTES + NB * (W_BYTES + B_BYTES) + 1024;
};
constexpr int TC_THREADS = 224;
constexpr int TC_SPIN_CAP = 1 << 24;

// ------------------------------------------------------------------ split + pack
// out: [3 terms][m_tiles][k_blocks][TC_TILE_BYTES]; rows >= M are zero.
// fp32 x[8] (8 consecutive k of one row) -> the three bf16 terms, stored at the operand-layout offset
__device__ __forceinline__ void tc_pack8(__nv_bfloat16 *out, size_t term_stride, int k_blocks, int row, int k8, const float (&x)[8]) {
	__align__(16) __nv_bfloat16 hi[8], mid[8], lo[8];
#pragma unroll
	for (int i = 0; i < 8; i++) {
		hi[i] = __float2bfloat16_rn(x[i]);
		const float r1 = x[i] - __bfloat162float(hi[i]);  // exact
		mid[i] = __float2bfloat16_rn(r1);
		const float r2 = r1 - __bfloat162float(mid[i]);   // exact
		lo[i] = __float2bfloat16_rn(r2);
	}
	const int mt = row / TC_BM, r = row % TC_BM, kb = (8 * k8) / TC_BK, kc = ((8 * k8) % TC_BK) / 8;
	const size_t off = (size_t(mt) * k_blocks + kb) * (TC_TILE_BYTES / 2) + (r / 8) * 256 + kc * 64 + (r % 8) * 8;
	*reinterpret_cast<uint4 *>(out + off) = *reinterpret_cast<const uint4 *>(hi);
	*reinterpret_cast<uint4 *>(out + term_stride + off) = *reinterpret_cast<const uint4 *>(mid);
	*reinterpret_cast<uint4 *>(out + 2 * term_stride + off) = *reinterpret_cast<const uint4 *>(lo);
}

// Work item c of a packing kernel -> (row, group of 8 consecutive k). Eight consecutive items are the eight rows
// of a core matrix at the same k group, so that a warp's 16-byte stores fill whole 128-byte lines of the packed
// tile (items in row-major order wrote every other 16 bytes of a line); each thread still reads 32 contiguous
// bytes of its row (one sector).
__device__ __forceinline__ void tc_chunk_to_row_k8(size_t c, int k8s, int &row, int &k8) {
	const size_t g = c / (size_t(8) * k8s);          // group of 8 rows
	const int w = int(c - g * (size_t(8) * k8s));    // item inside the group
	row = int(g) * 8 + (w & 7);
	k8 = w >> 3;
}

__global__ void __launch_bounds__(256) split_pack_kernel(const float *A, __nv_bfloat16 *out, int M, int K, int m_tiles) {
	pdl_trigger();
	pdl_wait();
	const int k_blocks = K / TC_BK;
	const size_t n_chunks = size_t(m_tiles) * TC_BM * (K / 8);  // one thread per (row, 8 consecutive k)
	const size_t term_stride = size_t(m_tiles) * k_blocks * (TC_TILE_BYTES / 2);
	for (size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x; c < n_chunks; c += size_t(gridDim.x) * blockDim.x) {
		int row, k8;
		tc_chunk_to_row_k8(c, K / 8, row, k8);
		float x[8];
		if (row < M) {
			const float4 a = *reinterpret_cast<const float4 *>(A + size_t(row) * K + 8 * k8);
			const float4 b = *reinterpret_cast<const float4 *>(A + size_t(row) * K + 8 * k8 + 4);
			x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
		} else {
#pragma unroll
			for (int i = 0; i < 8; i++) x[i] = 0.0f;
		}
		tc_pack8(out, term_stride, k_blocks, row, k8, x);
	}
}

// Residual + sandwich norms of one row, fused with the operand packing of the next GEMM:
//   if t:  h += rmsnorm(t; w_post)            (reference modules.hpp: post-norm, then the residual add)
//   if w_pre: pack( rmsnorm(h; w_pre) )       (the pre-norm of the following matmuls)
// One CTA of NT threads per row of the padded [m_tiles * 128] range (rows >= M are written as zeros). NT = 256:
// the sums run over d = tid, tid + 256, ... exactly like rmsnorm_rows_kernel, so the values are the ones the
// separate kernels produce. NT = 128 (thousands of rows): a row is a chain of dependent memory round trips and
// barriers that no amount of threads shortens, so the SM holds twice as many rows in flight instead.
// dim <= 2048, dim % 8 == 0.
// The branch output t is either a finished [M][dim] matrix (nsplit == 0) or the raw K-split partial
// sums of the GEMM that produced it: t[d] = tscale[d] * sum_sp tpart[(sp * M + row) * ldp + d], splits
// added in ascending order as the reduce kernel does.
template <int NT>
__global__ void __launch_bounds__(NT, NT == 128 ? 6 : 2) resnorm_pack_kernel(float *h, const float *t, const float *w_post, const float *w_pre,
                                                            __nv_bfloat16 *out, int M, int dim, int m_tiles, int nsplit,
                                                            int ldp, const float *tscale) {
	pdl_trigger();
	pdl_wait();
	constexpr int PER = 2048 / NT;         // values of a row per thread, at most
	constexpr int QB = NT == 256 ? 9 : 3;  // splits requested together (registers: the narrow variant wants six CTAs per SM)
	__shared__ float bred[NT / 32];
	__shared__ float row_s[2048];
	const int row = blockIdx.x, tid = threadIdx.x;
	const int k_blocks = dim / TC_BK;
	const size_t term_stride = size_t(m_tiles) * k_blocks * (TC_TILE_BYTES / 2);
	if (row >= M) {
		if (w_pre) {
			const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
			for (int k8 = tid; k8 < dim / 8; k8 += NT) tc_pack8(out, term_stride, k_blocks, row, k8, z);
		}
		return;
	}
	const size_t off = size_t(row) * dim;
	// The wide variant serves a few hundred rows, all resident at once: a row's time is its chain of dependent
	// memory round trips. Everything that does not depend on the partial sums (residual stream, norm weights,
	// column scales) is requested before them, not after the barriers that follow.
	constexpr bool PRE = NT == 256;
	float hv[PER], wp[PER], ts[PER];
	float4 wq0 = make_float4(0.f, 0.f, 0.f, 0.f), wq1 = wq0;
	if (PRE && t && nsplit > 0) {
#pragma unroll
		for (int j = 0; j < PER; j++) {
			const int d = tid + NT * j;
			hv[j] = wp[j] = ts[j] = 0.0f;
			if (d < dim) {
				hv[j] = h[off + d];
				wp[j] = w_post[d];
				ts[j] = tscale[d];
			}
		}
		if (w_pre && tid < dim / 8) {
			wq0 = *reinterpret_cast<const float4 *>(w_pre + 8 * tid);
			wq1 = *reinterpret_cast<const float4 *>(w_pre + 8 * tid + 4);
		}
	}
	if (t) {
		__shared__ float t_s[2048];
		float ss = 0.0f;
		if (nsplit > 0) {
			// Thread tid owns d = tid, tid + 256, ... (at most 8 values). The partial sums of up to nine splits
			// (the deepest split in use) for all of them are requested together: a row costs one L2 round
			// trip, not nsplit * 8. The splits are added in ascending order.
			float acc[PER];
#pragma unroll
			for (int j = 0; j < PER; j++) acc[j] = 0.0f;
			const size_t sstride = size_t(M) * ldp;
			const float *base = t + size_t(row) * ldp + tid;
			for (int s0 = 0; s0 < nsplit; s0 += QB) {
				float a[QB][PER];
#pragma unroll
				for (int q = 0; q < QB; q++)
#pragma unroll
					for (int j = 0; j < PER; j++)
						a[q][j] = (s0 + q < nsplit && tid + NT * j < dim) ? base[size_t(s0 + q) * sstride + NT * j] : 0.0f;
#pragma unroll
				for (int q = 0; q < QB; q++)
#pragma unroll
					for (int j = 0; j < PER; j++) acc[j] += a[q][j];
			}
#pragma unroll
			for (int j = 0; j < PER; j++) {
				const int d = tid + NT * j;
				if (d < dim) {
					const float v = acc[j] * (PRE ? ts[j] : tscale[d]);
					t_s[d] = v;
					ss = fmaf(v, v, ss);
				}
			}
		} else {
			for (int d = tid; d < dim; d += NT) {
				const float v = t[off + d];
				t_s[d] = v;
				ss = fmaf(v, v, ss);
			}
		}
		ss = block_sum<NT / 32>(ss, bred);
		const float r = inv_rms(ss, dim);
		if (PRE && nsplit > 0) {
#pragma unroll
			for (int j = 0; j < PER; j++) {
				const int d = tid + NT * j;
				if (d < dim) {
					const float y = (t_s[d] * r) * (wp[j] + 1.0f);
					const float hn = hv[j] + y;
					h[off + d] = hn;
					row_s[d] = hn;
				}
			}
		} else {
			for (int d = tid; d < dim; d += NT) {
				const float y = (t_s[d] * r) * (w_post[d] + 1.0f);
				const float hn = h[off + d] + y;
				h[off + d] = hn;
				row_s[d] = hn;
			}
		}
	} else {
		for (int d = tid; d < dim; d += NT) row_s[d] = h[off + d];
	}
	if (!w_pre) return;
	__syncthreads();
	float ss = 0.0f;
	for (int d = tid; d < dim; d += NT) {
		const float v = row_s[d];
		ss = fmaf(v, v, ss);
	}
	ss = block_sum<NT / 32>(ss, bred);
	const float r = inv_rms(ss, dim);
	if (PRE && t && nsplit > 0) {  // (dim / 8 <= 256: one group of eight per thread, its weights already here)
		if (tid < dim / 8) {
			const float wq[8] = {wq0.x, wq0.y, wq0.z, wq0.w, wq1.x, wq1.y, wq1.z, wq1.w};
			float x[8];
#pragma unroll
			for (int i = 0; i < 8; i++) x[i] = (row_s[8 * tid + i] * r) * (wq[i] + 1.0f);
			tc_pack8(out, term_stride, k_blocks, row, tid, x);
		}
		return;
	}
	for (int k8 = tid; k8 < dim / 8; k8 += NT) {
		float x[8];
#pragma unroll
		for (int i = 0; i < 8; i++) x[i] = (row_s[8 * k8 + i] * r) * (w_pre[8 * k8 + i] + 1.0f);
		tc_pack8(out, term_stride, k_blocks, row, k8, x);
	}
}

// GeGLU fused with the packing of the down projection's operand: pack( lut(gate) * up ), rows >= M zero
// With nsplit > 0, `up` points at the raw partial sums of the grouped up|gate GEMM (rows of 2K: up
// columns, then gate columns) and su / sg are the column scales; otherwise gate / up are finished.
__global__ void __launch_bounds__(256) geglu_pack_kernel(const float *gate, const float *up, __nv_bfloat16 *out, int M, int K,
                                                          int m_tiles, GeluLut lut, int nsplit, const float *su, const float *sg) {
	pdl_trigger();
	pdl_wait();
	const int k_blocks = K / TC_BK;
	const size_t n_chunks = size_t(m_tiles) * TC_BM * (K / 8);
	const size_t term_stride = size_t(m_tiles) * k_blocks * (TC_TILE_BYTES / 2);
	for (size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x; c < n_chunks; c += size_t(gridDim.x) * blockDim.x) {
		int row, k8;
		tc_chunk_to_row_k8(c, K / 8, row, k8);
		float x[8];
		if (row < M && nsplit > 0) {
			float4 u0 = make_float4(0.f, 0.f, 0.f, 0.f), u1 = u0, g0 = u0, g1 = u0;
			for (int s0 = 0; s0 < nsplit; s0 += 3) {  // three splits' loads in flight, added in split order
				float4 a0[3], a1[3], b0[3], b1[3];
#pragma unroll
				for (int q = 0; q < 3; q++) {
					const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
					a0[q] = a1[q] = b0[q] = b1[q] = z;
					if (s0 + q < nsplit) {
						const float *pr = up + (size_t(s0 + q) * M + row) * (2 * size_t(K)) + 8 * k8;
						a0[q] = *reinterpret_cast<const float4 *>(pr);
						a1[q] = *reinterpret_cast<const float4 *>(pr + 4);
						b0[q] = *reinterpret_cast<const float4 *>(pr + K);
						b1[q] = *reinterpret_cast<const float4 *>(pr + K + 4);
					}
				}
#pragma unroll
				for (int q = 0; q < 3; q++) {
					u0.x += a0[q].x; u0.y += a0[q].y; u0.z += a0[q].z; u0.w += a0[q].w;
					u1.x += a1[q].x; u1.y += a1[q].y; u1.z += a1[q].z; u1.w += a1[q].w;
					g0.x += b0[q].x; g0.y += b0[q].y; g0.z += b0[q].z; g0.w += b0[q].w;
					g1.x += b1[q].x; g1.y += b1[q].y; g1.z += b1[q].z; g1.w += b1[q].w;
				}
			}
			const float4 su0 = *reinterpret_cast<const float4 *>(su + 8 * k8), su1 = *reinterpret_cast<const float4 *>(su + 8 * k8 + 4);
			const float4 sg0 = *reinterpret_cast<const float4 *>(sg + 8 * k8), sg1 = *reinterpret_cast<const float4 *>(sg + 8 * k8 + 4);
			x[0] = lut(g0.x * sg0.x) * (u0.x * su0.x); x[1] = lut(g0.y * sg0.y) * (u0.y * su0.y);
			x[2] = lut(g0.z * sg0.z) * (u0.z * su0.z); x[3] = lut(g0.w * sg0.w) * (u0.w * su0.w);
			x[4] = lut(g1.x * sg1.x) * (u1.x * su1.x); x[5] = lut(g1.y * sg1.y) * (u1.y * su1.y);
			x[6] = lut(g1.z * sg1.z) * (u1.z * su1.z); x[7] = lut(g1.w * sg1.w) * (u1.w * su1.w);
		} else if (row < M) {
			const float4 g0 = *reinterpret_cast<const float4 *>(gate + size_t(row) * K + 8 * k8);
			const float4 g1 = *reinterpret_cast<const float4 *>(gate + size_t(row) * K + 8 * k8 + 4);
			const float4 u0 = *reinterpret_cast<const float4 *>(up + size_t(row) * K + 8 * k8);
			const float4 u1 = *reinterpret_cast<const float4 *>(up + size_t(row) * K + 8 * k8 + 4);
			x[0] = lut(g0.x) * u0.x; x[1] = lut(g0.y) * u0.y; x[2] = lut(g0.z) * u0.z; x[3] = lut(g0.w) * u0.w;
			x[4] = lut(g1.x) * u1.x; x[5] = lut(g1.y) * u1.y; x[6] = lut(g1.z) * u1.z; x[7] = lut(g1.w) * u1.w;
		} else {
#pragma unroll
			for (int i = 0; i < 8; i++) x[i] = 0.0f;
		}
		tc_pack8(out, term_stride, k_blocks, row, k8, x);
	}
}

// ------------------------------------------------------------------ tcgen05 helpers
// shared-memory matrix descriptor: K-major, no swizzle, LBO 128 B, SBO 512 B
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
	uint64_t d = 0;
	d |= uint64_t((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
	d |= uint64_t(128 >> 4) << 16;               // leading-dimension byte offset (next 8 k)
	d |= uint64_t(512 >> 4) << 32;               // stride-dimension byte offset (next 8 rows)
	d |= uint64_t(1) << 46;                      // descriptor version of this architecture
	return d;                                    // base offset 0, layout type 0 = no swizzle
}
// instruction descriptor: D fp32, A and B bf16, A K-major, B N-major (bit 16), M = 128, N = bn
__device__ __forceinline__ uint32_t tc_idesc(int bn) {
	return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (uint32_t(bn >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
	asm volatile(
	    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
	    "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
	    : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
	             "l"(src), "r"(bytes), "r"(smem_u32(bar))
	             : "memory");
}
// 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread (completion: tcgen05.wait::ld)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
	asm volatile(
	    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
	    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
	    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
	      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
	      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
	      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
	    : "r"(taddr)
	    : "memory");
}
__device__ __forceinline__ bool tc_wait(uint64_t *bar, uint32_t parity, int *err) {
	int spins = 0;
	while (!mbar_try_wait(bar, parity)) {
		if (++spins > TC_SPIN_CAP) {
			atomicExch(err, 6);
			return false;
		}
	}
	return true;
}

struct GemmTcArgs {
	const __nv_bfloat16 *apack;  // [3][m_tiles][k_blocks][8 KiB]
	// Up to three weight matrices with the same K share one launch and one packed A (q|k|v, up|gate):
	// group g owns the column tiles [tile_end[g-1], tile_end[g]) of the grid and columns col0[g].. of a
	// partial-sum row (N = total columns of all groups).
	int ngroups;
	int tile_end[3];
	int col0[3];
	int ncols[3];                // N_g (a multiple of 128; the last column tile of a group may reach past it)
	const float *scales[3];      // [N_g]
	float *C[3];                 // [M] rows of ldc[g] floats    (nsplit == 1: scaled result)
	int ldc[3];                  // row stride of C (>= N_g; lets a GEMM write a column block of a wider row)
	float *partial;              // [nsplit][M][N] raw sums      (nsplit > 1: summed and scaled by a second kernel)
	int M, N, K, m_tiles;
	int nsplit;                  // K-splits = gridDim.z; K / 32 must be a multiple of it
	int halves;                  // 2: this CTA's K range is accumulated in two TMEM accumulators (first / second half of its
	                             // K-blocks) that the epilogue adds in fp32 registers: halves the accumulation chain (the tensor
	                             // core truncates when it adds into the accumulator) without any partial-sum traffic. Else 1.
	int raw;                     // 1: always write raw partial sums (even unsplit); the consumer kernel adds the splits
	                             // and applies the column scales itself, so no reduce kernel runs
	unsigned *tickets;           // [gridDim.y * gridDim.x] zeros, or null. Non-null with nsplit > 1: the CTA that finishes
	                             // a tile last adds the partial sums in split order, scales and writes C itself
	unsigned long long *top1;    // non-null (nsplit == 1 only): no C is written; per row the largest scaled value and its column
	                             // are folded into top1[row] with atomicMax on tc_top1_key (lowest column on equal values)
	int top1_col0;               // added to a column index before it is recorded
	int *err;
};

// (value, column) -> a 64-bit key whose unsigned order is: larger value first, then the lower column. 0 = no candidate.
__device__ __forceinline__ unsigned long long tc_top1_key(float v, int col) {
	const uint32_t b = __float_as_uint(v);
	const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
	return (static_cast<unsigned long long>(ord) << 32) | static_cast<unsigned long long>(0xFFFFFFFFu - uint32_t(col));
}
// keys [M] -> maximum (or -inf) and column (or -1) per row
__global__ void top1_unpack_kernel(const unsigned long long *keys, int M, float *max_out, int *idx_out) {
	const int r = blockIdx.x * blockDim.x + threadIdx.x;
	if (r >= M) return;
	const unsigned long long k = keys[r];
	if (k == 0ull) {
		max_out[r] = -INFINITY;
		idx_out[r] = -1;
		return;
	}
	const uint32_t ord = uint32_t(k >> 32);
	max_out[r] = __uint_as_float((ord & 0x80000000u) ? (ord & 0x7FFFFFFFu) : ~ord);
	idx_out[r] = int(0xFFFFFFFFu - uint32_t(k));
}

template <int MT, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) qgemm_tc_kernel(const __grid_constant__ CUtensorMap wmap0,
                                                                 const __grid_constant__ CUtensorMap wmap1,
                                                                 const __grid_constant__ CUtensorMap wmap2, GemmTcArgs a) {
	using SH = TcShape<MT, BN>;
	constexpr int NA = SH::NA, NB = SH::NB;
	pdl_trigger();
	extern __shared__ uint8_t tc_smem_raw[];
	uint8_t *smem = reinterpret_cast<uint8_t *>((uintptr_t(tc_smem_raw) + 1023) & ~uintptr_t(1023));
	__shared__ uint64_t afull_bar[TcShape<MT, BN>::NA];  // A tiles of the stage landed (transaction bytes)
	__shared__ uint64_t afree_bar[TcShape<MT, BN>::NA];  // the MMAs that read the A stage have completed (tcgen05.commit)
	__shared__ uint64_t wfull_bar[TcShape<MT, BN>::NB];  // int8 W tile landed
	__shared__ uint64_t conv_bar[TcShape<MT, BN>::NB];   // W converted to bf16 (4 converter warps arrive)
	__shared__ uint64_t bfree_bar[TcShape<MT, BN>::NB];  // the MMAs that read the bf16 tile have completed
	__shared__ uint64_t acc_bar;               // all MMAs done: accumulators ready
	__shared__ uint32_t tmem_base_s;
	__shared__ int s_fail;
	__shared__ int s_issued_a, s_issued_w;  // k-blocks whose loads have been issued
	__shared__ int s_last, s_cnt;

	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int grp = (int(blockIdx.x) >= a.tile_end[0]) + (int(blockIdx.x) >= a.tile_end[1]);  // tile_end of unused groups = INT_MAX
	const int n0 = (int(blockIdx.x) - (grp == 0 ? 0 : (grp == 1 ? a.tile_end[0] : a.tile_end[1]))) * BN;  // column inside the group's matrix
	// (selects over constant indices: a run-time index into the parameter arrays would move them to local memory)
	const int pcol = (grp == 0 ? a.col0[0] : (grp == 1 ? a.col0[1] : a.col0[2])) + n0;  // column inside a partial-sum row
	const CUtensorMap *wmap = grp == 0 ? &wmap0 : (grp == 1 ? &wmap1 : &wmap2);
	float *const Cg = grp == 0 ? a.C[0] : (grp == 1 ? a.C[1] : a.C[2]);
	const float *const scg = grp == 0 ? a.scales[0] : (grp == 1 ? a.scales[1] : a.scales[2]);
	const int ldcg = grp == 0 ? a.ldc[0] : (grp == 1 ? a.ldc[1] : a.ldc[2]);
	const int ncg = grp == 0 ? a.ncols[0] : (grp == 1 ? a.ncols[1] : a.ncols[2]);
	const int mt0 = blockIdx.y * MT;
	const int nmt = min(MT, a.m_tiles - mt0);  // row tiles this CTA really has
	const int k_blocks_all = a.K / TC_BK;
	const int k_blocks = k_blocks_all / a.nsplit;   // this CTA's share of K
	const int kb_first = blockIdx.z * k_blocks;
	const size_t term_stride = size_t(a.m_tiles) * k_blocks_all * TC_TILE_BYTES;  // bytes

	if (tid == 0) {
		for (int s = 0; s < NA; s++) {
			mbar_init(&afull_bar[s], 1);
			mbar_init(&afree_bar[s], 1);
		}
		for (int s = 0; s < NB; s++) {
			mbar_init(&wfull_bar[s], 1);
			mbar_init(&conv_bar[s], 4);
			mbar_init(&bfree_bar[s], 1);
		}
		mbar_init(&acc_bar, 1);
		s_fail = 0;
		s_issued_a = 0;
		s_issued_w = 0;
		s_last = -1;
		s_cnt = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1) {  // TMEM: (MT row tiles) x (2 K halves) accumulators of BN fp32 columns = 512 columns
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512)
		             : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_base_s;

	auto stage_a = [&](int s, int term, int mt) { return smem + size_t(s) * SH::A_BYTES + (term * MT + mt) * TC_TILE_BYTES; };
	auto stage_w = [&](int s) { return smem + size_t(NA) * SH::A_BYTES + size_t(s) * SH::W_BYTES; };
	auto stage_b = [&](int s) { return smem + size_t(NA) * SH::A_BYTES + size_t(NB) * SH::W_BYTES + size_t(s) * SH::B_BYTES; };

	if (warp == 0) {
		// ------------------------------------------------------------ producer of the A stages
		if (lane == 0) {
			// The packed activations are the predecessor's output: wait for it here. The weight producer
			// (warp 6) does not wait: the weights are nobody's output, its first tiles land meanwhile. Everything
			// this CTA writes (C, partial sums, tickets) follows MMAs that need these A tiles, so it is ordered
			// behind the wait as well.
			pdl_wait();
			for (int kb = 0; kb < k_blocks; kb++) {
				const int s = kb % NA, use = kb / NA;
				if (use > 0 && !tc_wait(&afree_bar[s], (use - 1) & 1, a.err)) { s_fail = 1; break; }
				mbar_expect_tx(&afull_bar[s], uint32_t(3 * nmt * TC_TILE_BYTES));
				for (int term = 0; term < 3; term++)
					for (int mt = 0; mt < nmt; mt++) {
						const int mtg = mt0 + mt;
						const uint8_t *src = reinterpret_cast<const uint8_t *>(a.apack) + term * term_stride +
						                     (size_t(mtg) * k_blocks_all + kb_first + kb) * TC_TILE_BYTES;
						bulk_load(stage_a(s, term, mt), src, TC_TILE_BYTES, &afull_bar[s]);
					}
				s_issued_a = kb + 1;
			}
		}
	} else if (warp == 6) {
		// ------------------------------------------------------------ producer of the int8 W tiles
		if (lane == 0) {
			const uint64_t pol = l2_evict_first_policy();
			for (int kb = 0; kb < k_blocks; kb++) {
				const int s = kb % NB, use = kb / NB;
				// the slot's int8 tile was converted and its bf16 tile read by the MMAs of the previous use
				if (use > 0 && !tc_wait(&bfree_bar[s], (use - 1) & 1, a.err)) { s_fail = 1; break; }
				fence_proxy_async();
				mbar_expect_tx(&wfull_bar[s], uint32_t(SH::W_BYTES));
				tma_load_2d(stage_w(s), wmap, n0, (kb_first + kb) * TC_BK, &wfull_bar[s], pol);
				s_issued_w = kb + 1;
			}
		}
	} else if (warp == 1) {
		// ------------------------------------------------------------ MMA issuer
		if (lane == 0) {
			const uint32_t idesc = tc_idesc(BN);
			for (int kb = 0; kb < k_blocks; kb++) {
				const int sa = kb % NA, ua = kb / NA, sb = kb % NB, ub = kb / NB;
				if (!tc_wait(&conv_bar[sb], ub & 1, a.err) || !tc_wait(&afull_bar[sa], ua & 1, a.err)) { s_fail = 1; break; }
				tc_fence_after();
				const uint32_t b_addr = smem_u32(stage_b(sb));
				const int kb_half = (a.halves == 2) ? (k_blocks + 1) / 2 : k_blocks;  // first K-block of the second accumulator
				const bool second = kb >= kb_half;
				const bool first_of_acc = (kb == 0) || (kb == kb_half);
#pragma unroll
				for (int mt = 0; mt < MT; mt++) {
					if (mt < nmt) {  // (a predicate, not a break: the loop stays fully unrolled — one thread issues every MMA)
						const uint32_t d_tmem = tmem_base + uint32_t(mt * BN) + (second ? uint32_t(MT * BN) : 0u);
#pragma unroll
						for (int term = 0; term < 3; term++) {
							const uint32_t a_addr = smem_u32(stage_a(sa, term, mt));
#pragma unroll
							for (int j = 0; j < TC_BK / 16; j++) {
								const uint32_t acc = (!first_of_acc || term > 0 || j > 0) ? 1u : 0u;
								tc_mma(d_tmem, tc_smem_desc(a_addr + j * 256), tc_smem_desc(b_addr + j * 256), idesc, acc);
							}
						}
					}
				}
				// both arrive when the MMAs above have read their operands
				tc_commit(&afree_bar[sa]);
				tc_commit(&bfree_bar[sb]);
			}
			tc_commit(&acc_bar);
		}
	} else {
		// ------------------------------------------------------------ converters (warps 2..5, 128 threads)
		for (int kb = 0; kb < k_blocks; kb++) {
			const int s = kb % NB, use = kb / NB;
			// the slot's bf16 tile was last read by the MMAs of the previous use; the W producer waited for
			// them (bfree_bar) before it refilled the slot, so wfull_bar implies the tile may be overwritten
			bool ok = tc_wait(&wfull_bar[s], use & 1, a.err);
			if (!ok) { s_fail = 1; break; }
			const uint8_t *w = stage_w(s);
			uint8_t *b = stage_b(s);
			// The bf16 tile is N-major like W itself: a core matrix is 8 k-rows of 8 consecutive columns
			// (16 bytes each); byte offset of (k, n) = (n/8)*512 + (k/8)*128 + (k%8)*16 + (n%8)*2. One work
			// item = 8 consecutive int8 of one k-row (one 8-byte load) -> 8 bf16 (one 16-byte store). A warp
			// takes one group of 8 k-rows; its lanes cover the column groups, and the k-row of a lane rotates
			// with the lane index, so the loads (16 lanes: 16 different column groups) and the stores
			// (8 lanes: 8 different k-rows of a core matrix) are both free of bank conflicts.
			constexpr int G = BN / 8;        // column groups: 16 or 32
			constexpr int SUB = 32 / G;      // k-rows a warp covers per pass: 2 or 1
			const int kg = (warp - 2);       // this warp's group of 8 k-rows
			const int g = lane % G;
			uint2 raw[8 / SUB];
#pragma unroll
			for (int it = 0; it < 8 / SUB; it++) {
				const int kk = (g + it * SUB + lane / G) & 7;
				raw[it] = *reinterpret_cast<const uint2 *>(w + (kg * 8 + kk) * BN + 8 * g);
			}
#pragma unroll
			for (int it = 0; it < 8 / SUB; it++) {
				const int kk = (g + it * SUB + lane / G) & 7;
				__align__(16) __nv_bfloat162 v[4];
#pragma unroll
				for (int i = 0; i < 4; i++) {
					const uint32_t word = (i < 2) ? raw[it].x : raw[it].y;
					const uint32_t u0 = (word >> (16 * (i & 1))) & 0xFFu, u1 = (word >> (16 * (i & 1) + 8)) & 0xFFu;
					const float f0 = __uint_as_float(0x4B000000u | (u0 ^ 0x80u)) - 8388736.0f;
					const float f1 = __uint_as_float(0x4B000000u | (u1 ^ 0x80u)) - 8388736.0f;
					v[i] = __floats2bfloat162_rn(f0, f1);  // |int8| <= 128: exact in bf16
				}
				*reinterpret_cast<uint4 *>(b + g * 512 + kg * 128 + kk * 16) = *reinterpret_cast<const uint4 *>(v);
			}
			fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's reads
			__syncwarp();
			if (lane == 0) mbar_arrive(&conv_bar[s]);
		}
		// ------------------------------------------------------------ epilogue
		if (!*(volatile int *)&s_fail && tc_wait(&acc_bar, 0, a.err)) {
			tc_fence_after();
			const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
			// the operand rings are idle now (every load landed, every MMA read its operands): a corner of
			// them stages the output blocks, 32 x 36 floats per warp
			float *stg = reinterpret_cast<float *>(smem) + quad * (32 * 36);
			fence_proxy_async();
			const bool two = a.halves == 2 && k_blocks > 1;  // second accumulator in use
			const bool fin = a.nsplit == 1 && !a.raw;        // finished result (scaled); else raw partial sums
			constexpr int CH = BN / 32;                      // 32-column blocks per row tile
			// block e = (row tile e / CH, columns 32 * (e % CH) ..): request its accumulator(s) from TMEM
			auto request = [&](int e, uint32_t (&r)[32], uint32_t (&r2)[32]) {
				const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t((e / CH) * BN + (e % CH) * 32);
				tc_ld32(taddr, r);
				if (two) tc_ld32(taddr + uint32_t(MT * BN), r2);
			};
			float t1_best = -INFINITY;  // top-1 mode: this lane's row, running over the column blocks of one row tile
			int t1_col = -1;
			auto finish = [&](int e, uint32_t (&r)[32], uint32_t (&r2)[32]) {
				const int mt = e / CH, c = e % CH;
				if (two) {
#pragma unroll
					for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
				}
				if (a.top1) {
					// a lane holds 32 consecutive columns of one row: scan them in ascending order (strict >: the
					// lowest column of equal values stays), one atomicMax per row when the row tile is through
					if ((mt0 + mt) < a.m_tiles && n0 + c * 32 < ncg) {
						const float4 *sc = reinterpret_cast<const float4 *>(scg + n0 + c * 32);
#pragma unroll
						for (int i4 = 0; i4 < 8; i4++) {
							const float4 s4 = __ldg(sc + i4);
							const float v0 = __uint_as_float(r[4 * i4]) * s4.x, v1 = __uint_as_float(r[4 * i4 + 1]) * s4.y;
							const float v2 = __uint_as_float(r[4 * i4 + 2]) * s4.z, v3 = __uint_as_float(r[4 * i4 + 3]) * s4.w;
							const int cb = n0 + c * 32 + 4 * i4;
							if (v0 > t1_best) { t1_best = v0; t1_col = cb; }
							if (v1 > t1_best) { t1_best = v1; t1_col = cb + 1; }
							if (v2 > t1_best) { t1_best = v2; t1_col = cb + 2; }
							if (v3 > t1_best) { t1_best = v3; t1_col = cb + 3; }
						}
					}
					if (c == CH - 1) {
						const int row = (mt0 + mt) * TC_BM + quad * 32 + lane;
						if (row < a.M && t1_col >= 0) atomicMax(a.top1 + row, tc_top1_key(t1_best, a.top1_col0 + t1_col));
						t1_best = -INFINITY;
						t1_col = -1;
					}
					return;
				}
				if ((mt0 + mt) < a.m_tiles && n0 + c * 32 < ncg) {  // (a wide tile may reach past the group's last column)
					// A lane holds 32 consecutive columns of ONE row; written from here, a store instruction would
					// touch 32 rows (32 lines). The 32 x 32 block goes through shared memory instead (rows padded to
					// 36 floats: conflict-free both ways) and leaves as 8 instructions of 4 rows x 128 contiguous bytes.
#pragma unroll
					for (int i = 0; i < 32; i += 4)
						*reinterpret_cast<float4 *>(stg + lane * 36 + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
						                                                             __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
					__syncwarp();
					const int rsub = lane >> 3, c4 = lane & 7;
					// (raw partial sums are multiplied by 1.0f, which is exact)
					const float4 sc4 = fin ? *reinterpret_cast<const float4 *>(scg + n0 + c * 32 + 4 * c4) : make_float4(1.f, 1.f, 1.f, 1.f);
					float *dbase = fin ? Cg + n0 + c * 32 + 4 * c4 : a.partial + size_t(blockIdx.z) * a.M * a.N + pcol + c * 32 + 4 * c4;
					const size_t ld = fin ? size_t(ldcg) : size_t(a.N);
					const int row0 = (mt0 + mt) * TC_BM + quad * 32;
#pragma unroll
					for (int j = 0; j < 8; j++) {
						const int rr = j * 4 + rsub;
						float4 v = *reinterpret_cast<const float4 *>(stg + rr * 36 + 4 * c4);
						v.x *= sc4.x;
						v.y *= sc4.y;
						v.z *= sc4.z;
						v.w *= sc4.w;
						if (row0 + rr < a.M) *reinterpret_cast<float4 *>(dbase + size_t(row0 + rr) * ld) = v;
					}
					__syncwarp();
				}
			};
			// two register sets alternate: the TMEM load of the next block (~600 clk) runs under the stores of this one
			uint32_t ra[32], ra2[32], rb[32], rb2[32];
			const int ne = nmt * CH;  // even
			request(0, ra, ra2);
#pragma unroll 1
			for (int e = 0; e < ne; e += 2) {
				asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
				request(e + 1, rb, rb2);
				finish(e, ra, ra2);
				asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
				if (e + 2 < ne) request(e + 2, ra, ra2);
				finish(e + 1, rb, rb2);
			}
			if (a.nsplit > 1 && a.tickets && !a.raw) {
				// in-kernel split-K reduction: the CTA that arrives last at this tile's ticket sums the
				// partial tiles of all splits in split order (a fixed order: results are reproducible)
				// (the four epilogue warps meet through a shared counter and a bounded spin, never a
				// hardware barrier: a warp whose wait ran out must not be able to strand the others)
				__threadfence();
				__syncwarp();
				unsigned *tk = a.tickets + blockIdx.y * gridDim.x + blockIdx.x;
				if (lane == 0 && atomicAdd(&s_cnt, 1) == 3) {
					const unsigned t = atomicAdd(tk, 1u);
					*(volatile int *)&s_last = (t == unsigned(a.nsplit - 1)) ? 1 : 0;
				}
				int last = -1;
				for (int spins = 0; spins < TC_SPIN_CAP; spins++) {
					last = *(volatile int *)&s_last;
					if (last >= 0) break;
				}
				if (last < 0 && lane == 0) atomicExch(a.err, 7);
				if (last == 1) {
					__threadfence();
#pragma unroll 1
					for (int mt = 0; mt < nmt; mt++) {
						const int row = (mt0 + mt) * TC_BM + quad * 32 + lane;
						if (row >= a.M) continue;
#pragma unroll 1
						for (int c4 = 0; c4 < BN / 4; c4++) {
							if (n0 + 4 * c4 >= ncg) break;
							float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
							for (int s0 = 0; s0 < a.nsplit; s0 += 4) {
								float4 v[4];
#pragma unroll
								for (int q = 0; q < 4; q++) {
									v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
									if (s0 + q < a.nsplit)
										v[q] = __ldcg(reinterpret_cast<const float4 *>(a.partial + (size_t(s0 + q) * a.M + row) * a.N + pcol) + c4);
								}
#pragma unroll
								for (int q = 0; q < 4; q++) {
									sum.x += v[q].x;
									sum.y += v[q].y;
									sum.z += v[q].z;
									sum.w += v[q].w;
								}
							}
							const float4 sc = *reinterpret_cast<const float4 *>(scg + n0 + 4 * c4);
							*reinterpret_cast<float4 *>(Cg + size_t(row) * ldcg + n0 + 4 * c4) =
							    make_float4(sum.x * sc.x, sum.y * sc.y, sum.z * sc.z, sum.w * sc.w);
						}
					}
					__syncwarp();
					if (lane == 0 && atomicAdd(&s_cnt, 1) == 7) *tk = 0u;  // all four warps are done: ready for the next launch
				}
			}
		}
	}
	// ---------------------------------------------------------------- teardown
	tc_fence_before();
	__syncthreads();
	if (warp == 0 && lane == 0) {
		// every load that was issued must have landed before the shared memory is given up
		// (already true on the normal path; matters only after a wait ran out)
		const int ia = *(volatile int *)&s_issued_a, iw = *(volatile int *)&s_issued_w;
		for (int kb = max(0, ia - NA); kb < ia; kb++) {
			int spins = 0;
			while (!mbar_try_wait(&afull_bar[kb % NA], (kb / NA) & 1) && ++spins < TC_SPIN_CAP) {
			}
		}
		for (int kb = max(0, iw - NB); kb < iw; kb++) {
			int spins = 0;
			while (!mbar_try_wait(&wfull_bar[kb % NB], (kb / NB) & 1) && ++spins < TC_SPIN_CAP) {
			}
		}
	}
	if (warp == 1) {
		if (*(volatile int *)&s_fail && lane == 0) {
			// a wait ran out: let the MMAs in flight finish before the TMEM goes away
			int spins = 0;
			while (!mbar_try_wait(&acc_bar, 0) && ++spins < TC_SPIN_CAP) {
			}
		}
		__syncwarp();
		tc_fence_after();
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
	}
}

}  // namespace tg
