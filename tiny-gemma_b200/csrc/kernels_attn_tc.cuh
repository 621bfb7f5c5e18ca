// Prefill attention for long prompts on the 5th-generation tensor cores (tcgen05 + TMEM):
// causal / sliding-window softmax(q k^T / 16) v per (query, head), ops::attention_prefill
// (reference ops.hpp:377-526: a sliding-window query s sees keys max(0, s - window) .. s).
//
// The four heads share one KV head, so the (query, head) pairs of 32 consecutive queries form a 128-row
// operand: row r of tile t is query 32 t + r / 4, head r % 4 — the rows of q [S][4][256] as they lie.
// One CTA owns a row tile and walks its keys in tiles of 64:
//     S = Q K_j^T                    M128 x N64, contraction over the 256 head dimensions
//     online softmax on S            (running max m, sum l per row; one thread per row = one TMEM lane)
//     O = corr * O + P V_j           M128 x N256, contraction over the 64 keys
// fp32 accuracy on bf16 tensor cores as in the GEMM (kernels_gemm_tc.cuh): every fp32 operand is split into
// three bf16 terms x = hi + mid + lo and a product a * b is the six term products whose weight reaches
// 2^-24 (hi hi, hi mid, mid hi, mid mid, hi lo, lo hi), all accumulated in fp32 in TMEM.
//
// Operands are packed once per layer in the tensor core's shared-memory layouts (no swizzle, 8 x 8 core
// matrices), so that the CTA fetches them with plain bulk copies:
//     Q, K: split_pack_kernel ([3 terms][128-row tiles][8 blocks of 32 dimensions][8 KiB], K-major; a 64-key
//           tile is one half of a 128-row tile)
//     V:    attn_pack_v_kernel ([3 terms][32-key blocks][16 KiB], N-major like the GEMM's weight operand)
// Warps 0-3: softmax and epilogue (TMEM lanes 32 w ..); warp 4: one thread issues the bulk copies and the MMAs.
// Per key tile the ring carries eight Q|K blocks (one per 32 dimensions) and two V blocks (32 keys each);
// the V blocks land while the softmax runs. All waits are bounded; a wait that runs out sets *err, and the
// CTA lets its copies land and frees its TMEM before it returns.
#pragma once
#include "kernels_gemm_tc.cuh"

namespace tg {

constexpr int AT_TC_KT = 64;                       // keys per tile
constexpr int AT_TC_STAGE = 3 * 16384;             // ring stage: Q (3 x 8 KiB) + K (3 x 4 KiB), or V (3 x 16 KiB)
constexpr int AT_TC_NS = 3;                        // ring stages
constexpr int AT_TC_PBYTES = 3 * 2 * TC_TILE_BYTES;  // P: 3 terms x 2 blocks of 32 keys x [128][32] bf16
constexpr int AT_TC_SMEM = AT_TC_NS * AT_TC_STAGE + AT_TC_PBYTES + 1024;
constexpr int AT_TC_THREADS = 160;
constexpr int AT_TC_BLOCKS = 10;                   // ring blocks per key tile: 8 of Q|K, 2 of V

// v fp32 [S][256] -> three bf16 terms in the N-major operand layout, one 16 KiB tile per 32 keys:
// byte offset of (key k, dimension n) = (n / 8) * 512 + (k / 8) * 128 + (k % 8) * 16 + (n % 8) * 2. Keys >= S are zero.
__global__ void __launch_bounds__(256) attn_pack_v_kernel(const float *v, __nv_bfloat16 *out, int S, int nblocks) {
	pdl_trigger();
	pdl_wait();
	const size_t term_stride = size_t(nblocks) * 8192;  // elements
	const size_t n_items = size_t(nblocks) * 32 * 32;   // (key, 8 consecutive dimensions)
	for (size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x; c < n_items; c += size_t(gridDim.x) * blockDim.x) {
		const int key = int(c >> 5), n8 = int(c & 31);
		float x[8];
		if (key < S) {
			const float4 a = *reinterpret_cast<const float4 *>(v + size_t(key) * 256 + 8 * n8);
			const float4 b = *reinterpret_cast<const float4 *>(v + size_t(key) * 256 + 8 * n8 + 4);
			x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
		} else {
#pragma unroll
			for (int i = 0; i < 8; i++) x[i] = 0.0f;
		}
		__align__(16) __nv_bfloat16 hi[8], mid[8], lo[8];
#pragma unroll
		for (int i = 0; i < 8; i++) {
			hi[i] = __float2bfloat16_rn(x[i]);
			const float r1 = x[i] - __bfloat162float(hi[i]);
			mid[i] = __float2bfloat16_rn(r1);
			lo[i] = __float2bfloat16_rn(r1 - __bfloat162float(mid[i]));
		}
		const int kb = key >> 5, k = key & 31;
		const size_t off = size_t(kb) * 8192 + n8 * 256 + (k >> 3) * 64 + (k & 7) * 8;  // elements
		*reinterpret_cast<uint4 *>(out + off) = *reinterpret_cast<const uint4 *>(hi);
		*reinterpret_cast<uint4 *>(out + term_stride + off) = *reinterpret_cast<const uint4 *>(mid);
		*reinterpret_cast<uint4 *>(out + 2 * term_stride + off) = *reinterpret_cast<const uint4 *>(lo);
	}
}

// instruction descriptor: D fp32, A and B bf16, A K-major, B K-major (b_mn = 0) or N-major (1), M = 128, N = n
__device__ __forceinline__ uint32_t at_idesc(int n, int b_mn) {
	return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(b_mn) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
	asm volatile(
	    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
	    "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
	    "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
	    "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
	    "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
	    : "memory");
}
// bounded wait that also gives up when another role of the CTA already has
__device__ __forceinline__ bool at_wait(uint64_t *bar, uint32_t parity, int *err, volatile int *s_fail) {
	int spins = 0;
	while (!mbar_try_wait(bar, parity)) {
		if ((++spins & 1023) == 0 && *s_fail) return false;
		if (spins > TC_SPIN_CAP) {
			atomicExch(err, 6);
			*s_fail = 1;
			return false;
		}
	}
	return true;
}

struct AttnTcArgs {
	const __nv_bfloat16 *qp;  // [3][q_tiles][8][8 KiB]
	const __nv_bfloat16 *kp;  // [3][k_tiles][8][8 KiB]
	const __nv_bfloat16 *vp;  // [3][v_blocks][16 KiB]
	float *o;                 // [S][4][256]
	int S, q_tiles, k_tiles, v_blocks;
	int is_local, window;
	int *err;
};

__global__ void __launch_bounds__(AT_TC_THREADS, 1) attn_prefill_tc_kernel(AttnTcArgs a) {
	pdl_trigger();
	extern __shared__ uint8_t at_smem_raw[];
	uint8_t *smem = reinterpret_cast<uint8_t *>((uintptr_t(at_smem_raw) + 1023) & ~uintptr_t(1023));
	uint8_t *pbuf = smem + AT_TC_NS * AT_TC_STAGE;
	__shared__ uint64_t full_bar[AT_TC_NS];  // the stage's copies landed
	__shared__ uint64_t free_bar[AT_TC_NS];  // the MMAs that read the stage have completed
	__shared__ uint64_t s_bar;               // S = Q K^T of this key tile is complete (and every earlier MMA)
	__shared__ uint64_t p_bar;               // the four softmax warps wrote P and rescaled O
	__shared__ uint64_t o_bar;               // all MMAs done
	__shared__ uint32_t tmem_base_s;
	__shared__ int s_fail;

	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int tile = int(gridDim.x) - 1 - int(blockIdx.x);  // the tiles with the most keys start first
	const int q0 = tile * 32;                                // first query of the tile
	const int q_hi = min(a.S - 1, q0 + 31);
	// key tiles this row tile needs
	const int j_lo = a.is_local ? max(0, q0 - a.window) / AT_TC_KT : 0;
	const int j_hi = q_hi / AT_TC_KT;
	const int ntiles = j_hi - j_lo + 1;

	if (tid == 0) {
		for (int s = 0; s < AT_TC_NS; s++) {
			mbar_init(&full_bar[s], 1);
			mbar_init(&free_bar[s], 1);
		}
		mbar_init(&s_bar, 1);
		mbar_init(&p_bar, 4);
		mbar_init(&o_bar, 1);
		s_fail = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 4) {  // TMEM: S in columns 0..63, O in columns 128..383
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 128u;
	volatile int *fail = &s_fail;

	if (warp == 4) {
		// ------------------------------------------------------------ copies and MMAs (one thread)
		if (lane == 0) {
			pdl_wait();  // the packed operands are the predecessors' output
			const uint32_t idesc_qk = at_idesc(AT_TC_KT, 0), idesc_pv = at_idesc(256, 1);
			const size_t q_term = size_t(a.q_tiles) * 8 * TC_TILE_BYTES, k_term = size_t(a.k_tiles) * 8 * TC_TILE_BYTES,
			             v_term = size_t(a.v_blocks) * 16384;  // bytes
			const uint8_t *qp = reinterpret_cast<const uint8_t *>(a.qp), *kp = reinterpret_cast<const uint8_t *>(a.kp),
			              *vp = reinterpret_cast<const uint8_t *>(a.vp);
			const int total = ntiles * AT_TC_BLOCKS;
			// ring block g: key tile j_lo + g / 10; i = g % 10 < 8: the Q|K block of dimensions 32 i ..; else V block i - 8
			auto issue_load = [&](int g) -> bool {
				const int st = g % AT_TC_NS, use = g / AT_TC_NS;
				if (use > 0 && !at_wait(&free_bar[st], (use - 1) & 1, a.err, fail)) return false;
				const int j = j_lo + g / AT_TC_BLOCKS, i = g % AT_TC_BLOCKS;
				uint8_t *dst = smem + size_t(st) * AT_TC_STAGE;
				if (i < 8) {
					mbar_expect_tx(&full_bar[st], 3u * TC_TILE_BYTES + 3u * (TC_TILE_BYTES / 2));
					for (int t = 0; t < 3; t++) {
						bulk_load(dst + t * TC_TILE_BYTES, qp + t * q_term + (size_t(tile) * 8 + i) * TC_TILE_BYTES, TC_TILE_BYTES, &full_bar[st]);
						bulk_load(dst + 3 * TC_TILE_BYTES + t * (TC_TILE_BYTES / 2),
						          kp + t * k_term + (size_t(j >> 1) * 8 + i) * TC_TILE_BYTES + (j & 1) * (TC_TILE_BYTES / 2), TC_TILE_BYTES / 2,
						          &full_bar[st]);
					}
				} else {
					mbar_expect_tx(&full_bar[st], 3u * 16384u);
					for (int t = 0; t < 3; t++)
						bulk_load(dst + t * 16384, vp + t * v_term + (size_t(2 * j + (i - 8))) * 16384, 16384, &full_bar[st]);
				}
				return true;
			};
			bool ok = true;
			for (int g = 0; g < AT_TC_NS - 1 && g < total && ok; g++) ok = issue_load(g);
			// the six term products (A term, B term)
			const int ta[6] = {0, 0, 1, 1, 0, 2}, tb[6] = {0, 1, 0, 1, 2, 0};
			for (int g = 0; g < total && ok; g++) {
				const int i = g % AT_TC_BLOCKS, jt = g / AT_TC_BLOCKS;
				if (g + AT_TC_NS - 1 < total) ok = issue_load(g + AT_TC_NS - 1);
				if (!ok) break;
				if (i == 8 && !at_wait(&p_bar, jt & 1, a.err, fail)) { ok = false; break; }  // P written, O rescaled
				const int st = g % AT_TC_NS, use = g / AT_TC_NS;
				if (!at_wait(&full_bar[st], use & 1, a.err, fail)) { ok = false; break; }
				tc_fence_after();
				const uint32_t base = smem_u32(smem + size_t(st) * AT_TC_STAGE);
				if (i < 8) {
#pragma unroll
					for (int c = 0; c < 6; c++) {
						const uint32_t qa = base + ta[c] * TC_TILE_BYTES, kb_ = base + 3 * TC_TILE_BYTES + tb[c] * (TC_TILE_BYTES / 2);
#pragma unroll
						for (int j2 = 0; j2 < 2; j2++)
							tc_mma(tmem_s, tc_smem_desc(qa + j2 * 256), tc_smem_desc(kb_ + j2 * 256), idesc_qk, (i > 0 || c > 0 || j2 > 0) ? 1u : 0u);
					}
					tc_commit(&free_bar[st]);
					if (i == 7) tc_commit(&s_bar);
				} else {
					const int vb = i - 8;
					const uint32_t pb = smem_u32(pbuf);
#pragma unroll
					for (int c = 0; c < 6; c++) {
						const uint32_t pa = pb + (ta[c] * 2 + vb) * TC_TILE_BYTES, vv = base + tb[c] * 16384;
#pragma unroll
						for (int j2 = 0; j2 < 2; j2++)
							tc_mma(tmem_o, tc_smem_desc(pa + j2 * 256), tc_smem_desc(vv + j2 * 256), idesc_pv, (jt > 0 || vb > 0 || c > 0 || j2 > 0) ? 1u : 0u);
					}
					tc_commit(&free_bar[st]);
				}
			}
			tc_commit(&o_bar);
		}
	} else {
		// ------------------------------------------------------------ softmax (thread = row = TMEM lane)
		const int r = tid;                         // row of the tile
		const int qi = q0 + (r >> 2);              // this row's query
		const bool row_ok = qi < a.S;
		const int k_min = a.is_local ? max(0, qi - a.window) : 0;
		const uint32_t lane_base = uint32_t(warp * 32) << 16;
		float m = -INFINITY, l = 0.0f;
		bool ok = true;
		for (int jt = 0; jt < ntiles && ok; jt++) {
			if (!at_wait(&s_bar, jt & 1, a.err, fail)) { ok = false; break; }
			tc_fence_after();
			uint32_t s0[32], s1[32];
			tc_ld32(tmem_s + lane_base, s0);
			tc_ld32(tmem_s + lane_base + 32u, s1);
			asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
			const int kbase = (j_lo + jt) * AT_TC_KT;
			float mt = -INFINITY;
#pragma unroll
			for (int c = 0; c < 64; c++) {
				const int key = kbase + c;
				const bool vis = row_ok && key <= qi && key >= k_min;
				float sv = __uint_as_float(c < 32 ? s0[c & 31] : s1[c & 31]) * 0.0625f;  // 1 / sqrt(256), exact
				sv = vis ? sv : -INFINITY;
				if (c < 32) s0[c & 31] = __float_as_uint(sv); else s1[c & 31] = __float_as_uint(sv);
				mt = fmaxf(mt, sv);
			}
			const float mn = fmaxf(m, mt);
			const bool none = mn == -INFINITY;            // no visible key so far
			const float corr = none ? 1.0f : expf(m - mn);  // exp(-inf) = 0 at the row's first visible tile
			float sum = 0.0f;
			// probabilities -> three bf16 terms in the A-operand layout: P[term][block of 32 keys] tiles of [128][32]
#pragma unroll
			for (int kc = 0; kc < 8; kc++) {  // 8 keys at a time
				__align__(16) __nv_bfloat16 hi[8], mid[8], lo[8];
#pragma unroll
				for (int u = 0; u < 8; u++) {
					const int c = 8 * kc + u;
					const float sv = __uint_as_float(c < 32 ? s0[c & 31] : s1[c & 31]);
					const float p = none ? 0.0f : expf(sv - mn);  // exp(-inf) = 0 for masked keys
					sum += p;
					hi[u] = __float2bfloat16_rn(p);
					const float r1 = p - __bfloat162float(hi[u]);
					mid[u] = __float2bfloat16_rn(r1);
					lo[u] = __float2bfloat16_rn(r1 - __bfloat162float(mid[u]));
				}
				const int vb = kc >> 2, k8 = kc & 3;
				uint8_t *dst = pbuf + vb * TC_TILE_BYTES + (r >> 3) * 512 + k8 * 128 + (r & 7) * 16;
				*reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(hi);
				*reinterpret_cast<uint4 *>(dst + 2 * TC_TILE_BYTES) = *reinterpret_cast<const uint4 *>(mid);
				*reinterpret_cast<uint4 *>(dst + 4 * TC_TILE_BYTES) = *reinterpret_cast<const uint4 *>(lo);
			}
			l = fmaf(l, corr, sum);
			m = mn;
			// O = corr * O (the previous tile's P V has completed: s_bar follows it in the issue order)
			if (jt > 0 && !__all_sync(0xffffffffu, corr == 1.0f)) {
#pragma unroll 1
				for (int c8 = 0; c8 < 8; c8++) {
					uint32_t ov[32];
					tc_ld32(tmem_o + lane_base + uint32_t(32 * c8), ov);
					asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
					for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
					tc_st32(tmem_o + lane_base + uint32_t(32 * c8), ov);
				}
				asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
			}
			fence_proxy_async();  // P: generic-proxy stores -> the tensor core's reads
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(&p_bar);
		}
		// ------------------------------------------------------------ epilogue: o = O / l
		if (ok && at_wait(&o_bar, 0, a.err, fail)) {
			tc_fence_after();
			const float inv = row_ok ? 1.0f / l : 0.0f;  // (a visible key always exists: the query itself)
			float *orow = a.o + (size_t(tile) * 128 + r) * 256;
#pragma unroll 1
			for (int c8 = 0; c8 < 8; c8++) {
				uint32_t ov[32];
				tc_ld32(tmem_o + lane_base + uint32_t(32 * c8), ov);
				asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
				if (row_ok) {
#pragma unroll
					for (int i = 0; i < 32; i += 4)
						*reinterpret_cast<float4 *>(orow + 32 * c8 + i) =
						    make_float4(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv, __uint_as_float(ov[i + 2]) * inv,
						                __uint_as_float(ov[i + 3]) * inv);
				}
			}
		}
	}
	// ---------------------------------------------------------------- teardown
	tc_fence_before();
	__syncthreads();
	if (*fail) {
		// a wait ran out: give the copies and MMAs in flight time to finish before shared memory and TMEM go away
		const long long t0 = clock64();
		while (clock64() - t0 < 2000000) {
		}
		__syncthreads();
	}
	if (warp == 4) {
		__syncwarp();
		tc_fence_after();
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(512) : "memory");
	}
}

}  // namespace tg
