// Prefill attention for long prompts on the 5th-generation tensor cores (tcgen05 + TMEM):
// causal / sliding-window softmax(q k^T / 16) v per (query, head), ops::attention_prefill
// (reference ops.hpp:377-526: a sliding-window query s sees keys max(0, s - window) .. s).
//
// The four heads share one KV head, so the (query, head) pairs of 32 consecutive queries form a 128-row
// operand: row r of tile t is query 32 t + r / 4, head r % 4 — the rows of q [S][4][256] as they lie.
// One CTA owns a row tile and walks its keys in tiles of 64:
//     S = Q K_j^T                    M128 x N64, contraction over the 256 head dimensions
//     online softmax on S            (max in use m and sum l per row; a row = one TMEM lane, two threads)
//     O = corr * O + P V_j           M128 x N256, contraction over the 64 keys
// fp32 accuracy on bf16 tensor cores as in the GEMM (kernels_gemm_tc.cuh): every fp32 operand is split into
// three bf16 terms x = hi + mid + lo and a product a * b is the six term products whose weight reaches
// 2^-24 (hi hi, hi mid, mid hi, mid mid, hi lo, lo hi), all accumulated in fp32 in TMEM.
//
// Operands are packed once per layer in the tensor core's shared-memory layouts (no swizzle, 8 x 8 core
// matrices), so that the CTA fetches them with plain bulk copies:
//     Q, K: split_pack_kernel ([3 terms][128-row tiles][8 blocks of 32 dimensions][8 KiB], K-major; a 64-key
//           tile is one half of a 128-row tile)
//     V:    attn_pack_v_kernel ([3 terms][16-key blocks][8 KiB], N-major like the GEMM's weight operand)
// Warps 0-7: softmax and epilogue (two threads per row: warps w and w + 4 share the TMEM lanes 32 (w % 4) ..
// and take half of a tile's keys each); warp 8: one thread issues the MMAs; warp 9: one thread issues the bulk
// copies, up to four ring blocks ahead of the MMAs.
// Per key tile the ring carries eight Q|K blocks (one per 32 dimensions) and four V blocks (16 keys each).
// S is double-buffered in TMEM and the MMAs are issued as Q K_0^T, Q K_1^T, P V_0, Q K_2^T, P V_1, ...: while the
// softmax warps work on tile t the tensor core runs Q K_{t+1}^T and P V_{t-1}. The running max is only moved (and
// O rescaled, a TMEM round trip) when a row's new max exceeds the one in use by more than 8: the probabilities
// are then at most e^8, far inside fp32, and the final division by the row sum removes the common factor.
// All waits are bounded; a wait that runs out sets *err, and the CTA lets its copies land and frees its
// TMEM before it returns.
#pragma once
#include "kernels_gemm_tc.cuh"

namespace tg {

constexpr int AT_TC_KT = 64;                       // keys per tile
constexpr int AT_TC_STAGE = 36 * 1024;             // ring stage: Q (3 x 8 KiB) + K (3 x 4 KiB), or V (3 x 8 KiB)
constexpr int AT_TC_NS = 4;                        // ring stages
constexpr int AT_TC_PBYTES = 3 * 2 * TC_TILE_BYTES;  // P: 3 terms x 2 blocks of 32 keys x [128][32] bf16
constexpr int AT_TC_SMEM = AT_TC_NS * AT_TC_STAGE + AT_TC_PBYTES + 1024;
constexpr int AT_TC_THREADS = 320;                 // 8 softmax warps, the MMA-issuing warp, the copy-issuing warp
constexpr int AT_TC_BLOCKS = 12;                   // ring blocks per key tile: 8 of Q|K (32 dimensions each), 4 of V (16 keys each)
constexpr int AT_TC_VBYTES = 8192;                 // one term of a V block: [16 keys][256 dimensions] bf16

// v fp32 [S][256] -> three bf16 terms in the N-major operand layout, one 8 KiB tile per 16 keys (one MMA K-step):
// byte offset of (key k, dimension n) = (n / 8) * 256 + (k / 8) * 128 + (k % 8) * 16 + (n % 8) * 2. Keys >= S are zero.
__global__ void __launch_bounds__(256) attn_pack_v_kernel(const float *v, __nv_bfloat16 *out, int S, int nblocks) {
	pdl_trigger();
	pdl_wait();
	const size_t term_stride = size_t(nblocks) * 4096;  // elements
	const size_t n_items = size_t(nblocks) * 16 * 32;   // (key, 8 consecutive dimensions)
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
		const int kb = key >> 4, k = key & 15;
		const size_t off = size_t(kb) * 4096 + n8 * 128 + (k >> 3) * 64 + (k & 7) * 8;  // elements
		*reinterpret_cast<uint4 *>(out + off) = *reinterpret_cast<const uint4 *>(hi);
		*reinterpret_cast<uint4 *>(out + term_stride + off) = *reinterpret_cast<const uint4 *>(mid);
		*reinterpret_cast<uint4 *>(out + 2 * term_stride + off) = *reinterpret_cast<const uint4 *>(lo);
	}
}

// instruction descriptor: D fp32, A and B bf16, A K-major, B K-major (b_mn = 0) or N-major (1), M = 128, N = n
__device__ __forceinline__ uint32_t at_idesc(int n, int b_mn) {
	return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(b_mn) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);
}
// shared-memory matrix descriptor of a V block: no swizzle, 128 B between the two 8-key groups, 256 B between
// groups of 8 dimensions
__device__ __forceinline__ uint64_t at_vdesc(uint32_t smem_addr) {
	uint64_t d = 0;
	d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
	d |= uint64_t(128 >> 4) << 16;
	d |= uint64_t(256 >> 4) << 32;
	d |= uint64_t(1) << 46;
	return d;
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

// The two threads of a row hand each other one float through shared memory: value, then tag; the reader
// polls the partner's tag (bounded like every wait here).
__device__ __forceinline__ bool at_exchange(float *val, int *tag, int me, float v, int t, float *other, int *err, volatile int *s_fail) {
	volatile float *xv = val;
	volatile int *xg = tag;
	xv[me] = v;
	__threadfence_block();
	xg[me] = t;
	int spins = 0;
	while (xg[me ^ 1] != t) {
		if ((++spins & 1023) == 0 && *s_fail) return false;
		if (spins > TC_SPIN_CAP) {
			atomicExch(err, 6);
			*s_fail = 1;
			return false;
		}
	}
	__threadfence_block();
	*other = xv[me ^ 1];
	return true;
}

struct AttnTcArgs {
	const __nv_bfloat16 *qp;  // [3][q_tiles][8][8 KiB]
	const __nv_bfloat16 *kp;  // [3][k_tiles][8][8 KiB]
	const __nv_bfloat16 *vp;  // [3][v_blocks][8 KiB]
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
	__shared__ uint64_t s_bar[2];            // S = Q K^T of a key tile is complete (two S buffers, tiles alternate)
	__shared__ uint64_t p_bar;               // the eight softmax warps wrote P and rescaled O
	__shared__ uint64_t pv_bar;              // P V of a key tile is complete: P may be overwritten, O read
	__shared__ uint64_t o_bar;               // all MMAs done
	__shared__ uint32_t tmem_base_s;
	__shared__ int s_fail;
	__shared__ float xm[2][128][2];          // half-row maxima (by tile parity), row sums at the end
	__shared__ int xt[2][128][2];            // their tags: the exchange between the two threads of a row is a bounded poll

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
		mbar_init(&s_bar[0], 1);
		mbar_init(&s_bar[1], 1);
		mbar_init(&p_bar, 8);
		mbar_init(&pv_bar, 1);
		mbar_init(&o_bar, 1);
		s_fail = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	for (int i = tid; i < 2 * 128 * 2; i += AT_TC_THREADS) (&xt[0][0][0])[i] = 0;
	if (warp == 8) {  // TMEM: S in columns 0..63 and 64..127 (alternating tiles), O in columns 128..383
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 128u;
	volatile int *fail = &s_fail;

	// MMA order: QK(0), then for t = 1 .. n: QK(t) (if t < n), PV(t - 1). Ring block g in that order:
	// g < 8: QK(0) block g; else g' = g - 8, t = 1 + g' / 12, r = g' % 12: QK(t) block r (r < 8, t < n) or PV(t - 1)
	// block r - 8 (t < n), and the last four blocks are PV(n - 1).
	struct Blk {
		int qk, tile, i;  // qk: 1 = Q|K block i (dimensions 32 i ..) of key tile `tile`, 0 = V block i (keys 16 i ..) of it
	};
	auto blk = [&](int g) -> Blk {
		if (g < 8) return Blk{1, 0, g};
		const int gp = g - 8, t = 1 + gp / AT_TC_BLOCKS, r = gp % AT_TC_BLOCKS;
		if (t >= ntiles) return Blk{0, ntiles - 1, r};
		return r < 8 ? Blk{1, t, r} : Blk{0, t - 1, r - 8};
	};
	const int total = ntiles * AT_TC_BLOCKS;
	if (warp == 9) {
		// ------------------------------------------------------------ bulk copies (one thread), up to AT_TC_NS blocks ahead
		if (lane == 0) {
			pdl_wait();  // the packed operands are the predecessors' output
			const size_t q_term = size_t(a.q_tiles) * 8 * TC_TILE_BYTES, k_term = size_t(a.k_tiles) * 8 * TC_TILE_BYTES,
			             v_term = size_t(a.v_blocks) * AT_TC_VBYTES;  // bytes
			const uint8_t *qp = reinterpret_cast<const uint8_t *>(a.qp), *kp = reinterpret_cast<const uint8_t *>(a.kp),
			              *vp = reinterpret_cast<const uint8_t *>(a.vp);
			for (int g = 0; g < total; g++) {
				const int st = g % AT_TC_NS, use = g / AT_TC_NS;
				if (use > 0 && !at_wait(&free_bar[st], (use - 1) & 1, a.err, fail)) break;
				const Blk b = blk(g);
				const int j = j_lo + b.tile, i = b.i;
				uint8_t *dst = smem + size_t(st) * AT_TC_STAGE;
				if (b.qk) {
					mbar_expect_tx(&full_bar[st], 3u * TC_TILE_BYTES + 3u * (TC_TILE_BYTES / 2));
					for (int t = 0; t < 3; t++) {
						bulk_load(dst + t * TC_TILE_BYTES, qp + t * q_term + (size_t(tile) * 8 + i) * TC_TILE_BYTES, TC_TILE_BYTES, &full_bar[st]);
						bulk_load(dst + 3 * TC_TILE_BYTES + t * (TC_TILE_BYTES / 2),
						          kp + t * k_term + (size_t(j >> 1) * 8 + i) * TC_TILE_BYTES + (j & 1) * (TC_TILE_BYTES / 2), TC_TILE_BYTES / 2,
						          &full_bar[st]);
					}
				} else {
					mbar_expect_tx(&full_bar[st], 3u * AT_TC_VBYTES);
					for (int t = 0; t < 3; t++)
						bulk_load(dst + t * AT_TC_VBYTES, vp + t * v_term + (size_t(4 * j + i)) * AT_TC_VBYTES, AT_TC_VBYTES, &full_bar[st]);
				}
			}
		}
	} else if (warp == 8) {
		// ------------------------------------------------------------ MMAs (one thread)
		if (lane == 0) {
			const uint32_t idesc_qk = at_idesc(AT_TC_KT, 0), idesc_pv = at_idesc(256, 1);
			// the six term products (A term, B term)
			const int ta[6] = {0, 0, 1, 1, 0, 2}, tb[6] = {0, 1, 0, 1, 2, 0};
			bool ok = true;
			for (int g = 0; g < total && ok; g++) {
				const Blk b = blk(g);
				if (!b.qk && b.i == 0 && !at_wait(&p_bar, b.tile & 1, a.err, fail)) { ok = false; break; }  // P written, O rescaled
				const int st = g % AT_TC_NS, use = g / AT_TC_NS;
				if (!at_wait(&full_bar[st], use & 1, a.err, fail)) { ok = false; break; }
				tc_fence_after();
				const uint32_t base = smem_u32(smem + size_t(st) * AT_TC_STAGE);
				if (b.qk) {
					const uint32_t d_s = tmem_s + uint32_t((b.tile & 1) * AT_TC_KT);
#pragma unroll
					for (int c = 0; c < 6; c++) {
						const uint32_t qa = base + ta[c] * TC_TILE_BYTES, kb_ = base + 3 * TC_TILE_BYTES + tb[c] * (TC_TILE_BYTES / 2);
#pragma unroll
						for (int j2 = 0; j2 < 2; j2++)
							tc_mma(d_s, tc_smem_desc(qa + j2 * 256), tc_smem_desc(kb_ + j2 * 256), idesc_qk, (b.i > 0 || c > 0 || j2 > 0) ? 1u : 0u);
					}
					tc_commit(&free_bar[st]);
					if (b.i == 7) tc_commit(&s_bar[b.tile & 1]);
				} else {
					const int vb = b.i;  // keys 16 vb ..: K-step vb % 2 of P's 32-key block vb / 2
					const uint32_t pb = smem_u32(pbuf);
#pragma unroll
					for (int c = 0; c < 6; c++) {
						const uint32_t pa = pb + (ta[c] * 2 + (vb >> 1)) * TC_TILE_BYTES + (vb & 1) * 256, vv = base + tb[c] * AT_TC_VBYTES;
						tc_mma(tmem_o, tc_smem_desc(pa), at_vdesc(vv), idesc_pv, (b.tile > 0 || vb > 0 || c > 0) ? 1u : 0u);
					}
					tc_commit(&free_bar[st]);
					if (vb == 3) tc_commit(&pv_bar);
				}
			}
			tc_commit(&o_bar);
		}
	} else {
		// ------------------------------------------------------------ softmax (two threads per row = TMEM lane)
		// warps w and w + 4 share the TMEM lanes 32 (w % 4) ..: thread (w, lane) owns row 32 (w % 4) + lane and the
		// 32 keys 32 (w / 4) .. of every tile (= one of P's two 32-key blocks), and half of O's columns
		const int qd = warp & 3, hf = warp >> 2;
		const int r = qd * 32 + lane;              // row of the tile
		const int qi = q0 + (r >> 2);              // this row's query
		const bool row_ok = qi < a.S;
		const int k_min = a.is_local ? max(0, qi - a.window) : 0;
		const uint32_t lane_base = uint32_t(qd * 32) << 16;
		float m = -INFINITY, l = 0.0f;             // max in use (the same in both threads of a row), sum over this thread's keys
		bool ok = true;
		for (int jt = 0; jt < ntiles && ok; jt++) {
			if (!at_wait(&s_bar[jt & 1], (jt >> 1) & 1, a.err, fail)) { ok = false; break; }
			tc_fence_after();
			uint32_t sv[32];
			tc_ld32(tmem_s + lane_base + uint32_t((jt & 1) * AT_TC_KT + 32 * hf), sv);
			asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
			const int kbase = (j_lo + jt) * AT_TC_KT + 32 * hf;
			// (most tiles lie wholly inside every row's key range: no per-key test there)
			const bool all_vis = (j_lo + jt) * AT_TC_KT + AT_TC_KT - 1 <= q0 && (!a.is_local || (j_lo + jt) * AT_TC_KT >= q0 + 31 - a.window);
			float mt = -INFINITY;
			if (all_vis) {
#pragma unroll
				for (int c = 0; c < 32; c++) {
					const float x = __uint_as_float(sv[c]) * 0.0625f;  // 1 / sqrt(256), exact
					sv[c] = __float_as_uint(x);
					mt = fmaxf(mt, x);
				}
			} else {
#pragma unroll
				for (int c = 0; c < 32; c++) {
					const int key = kbase + c;
					const bool vis = row_ok && key <= qi && key >= k_min;
					const float x = vis ? __uint_as_float(sv[c]) * 0.0625f : -INFINITY;
					sv[c] = __float_as_uint(x);
					mt = fmaxf(mt, x);
				}
			}
			// the row's max over both halves
			{
				float other;
				if (!at_exchange(xm[jt & 1][r], xt[jt & 1][r], hf, mt, jt + 1, &other, a.err, fail)) { ok = false; break; }
				mt = fmaxf(mt, other);
			}
			// the max in use moves only when the new one exceeds it by more than 8 (or at the row's first visible key)
			const float mn = (mt > m + 8.0f || m == -INFINITY) ? fmaxf(m, mt) : m;
			const bool none = mn == -INFINITY;            // no visible key so far
			const float corr = none ? 1.0f : expf(m - mn);  // exp(-inf) = 0 at the row's first visible tile; 1 when the max stays
			// probabilities and their three bf16 terms by truncation (p >= 0; hi + mid + lo = p exactly: 8 + 8 + 8 bits)
			float sum = 0.0f;
			uint32_t ph[16], pm[16], pl[16];  // bf16 pairs
#pragma unroll
			for (int c = 0; c < 32; c += 2) {
				uint32_t hb[2], mb[2], lb[2];
#pragma unroll
				for (int u = 0; u < 2; u++) {
					const float pv = none ? 0.0f : expf(__uint_as_float(sv[c + u]) - mn);  // exp(-inf) = 0 for masked keys
					sum += pv;
					hb[u] = __float_as_uint(pv) & 0xFFFF0000u;
					const float r1 = pv - __uint_as_float(hb[u]);
					mb[u] = __float_as_uint(r1) & 0xFFFF0000u;
					lb[u] = __float_as_uint(r1 - __uint_as_float(mb[u]));  // at most 8 significant bits: exact in bf16
				}
				ph[c / 2] = __byte_perm(hb[0], hb[1], 0x7632);
				pm[c / 2] = __byte_perm(mb[0], mb[1], 0x7632);
				pl[c / 2] = __byte_perm(lb[0], lb[1], 0x7632);
			}
			l = fmaf(l, corr, sum);
			m = mn;
			// the previous tile's P V reads P (and accumulates into O) until pv_bar: wait for it before touching either
			if (jt > 0 && !at_wait(&pv_bar, (jt - 1) & 1, a.err, fail)) { ok = false; break; }
			tc_fence_after();
			// P[term][block hf] tiles of [128][32] in the A-operand layout
#pragma unroll
			for (int k8 = 0; k8 < 4; k8++) {
				uint8_t *dst = pbuf + hf * TC_TILE_BYTES + (r >> 3) * 512 + k8 * 128 + (r & 7) * 16;
				*reinterpret_cast<uint4 *>(dst) = make_uint4(ph[4 * k8], ph[4 * k8 + 1], ph[4 * k8 + 2], ph[4 * k8 + 3]);
				*reinterpret_cast<uint4 *>(dst + 2 * TC_TILE_BYTES) = make_uint4(pm[4 * k8], pm[4 * k8 + 1], pm[4 * k8 + 2], pm[4 * k8 + 3]);
				*reinterpret_cast<uint4 *>(dst + 4 * TC_TILE_BYTES) = make_uint4(pl[4 * k8], pl[4 * k8 + 1], pl[4 * k8 + 2], pl[4 * k8 + 3]);
			}
			// O = corr * O: this thread's half of the row's 256 columns
			if (jt > 0 && !__all_sync(0xffffffffu, corr == 1.0f)) {
#pragma unroll 1
				for (int c8 = 4 * hf; c8 < 4 * hf + 4; c8++) {
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
			float l_other = 0.0f;  // (the partner is past its last read of slot 0: it arrived at p_bar, which o_bar follows)
			const bool got = at_exchange(xm[0][r], xt[0][r], hf, l, 0x40000000, &l_other, a.err, fail);
			const float lt = l + l_other;
			const float inv = (row_ok && got) ? 1.0f / lt : 0.0f;  // (a visible key always exists: the query itself)
			float *orow = a.o + (size_t(tile) * 128 + r) * 256;
#pragma unroll 1
			for (int c8 = 4 * hf; c8 < 4 * hf + 4; c8++) {
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
	if (warp == 8) {
		__syncwarp();
		tc_fence_after();
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(512) : "memory");
	}
}

}  // namespace tg
