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

// Row-wise (max, argmax) over a slice of the vocabulary: rows [M][ncols] hold the logits of
// columns col0.. of M sequences; writes the maximum and its GLOBAL index (col0 + local), lowest
// index on ties (the rule of ops::argmax_logits). One CTA per row.
__global__ void __launch_bounds__(SM_THREADS) top1_rows_kernel(const float *logits, int ncols, int col0, float *max_out,
                                                               int *idx_out) {
	__shared__ float sv[SM_NWARPS];
	__shared__ int si[SM_NWARPS];
	const int r = blockIdx.x, tid = threadIdx.x;
	const float *x = logits + size_t(r) * ncols;
	float best = -INFINITY;
	int arg = -1;
	for (int i = tid; i < ncols; i += SM_THREADS) {
		float v = x[i];
		if (v > best) { best = v; arg = i; }
	}
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
		max_out[r] = best;
		idx_out[r] = arg < 0 ? -1 : col0 + arg;
	}
}

// ops::minp_logits, reference ops.hpp:762-859.
//  (1) x /= temp  (2) rowmax  (3) p = exp(x - rowmax), maxp  (4) cut = minp*maxp,
//  denom = sum of p >= cut  (5) every p *= 1/denom — tokens under the cut keep
//  their mass, only the denominator is masked  (6) first index whose running
//  fp32 sum reaches randf, else 0.
// Steps 1-5 are data-parallel. Step 6 must reproduce a *sequential* fp32 sum
// (fp32 addition is not associative, and the crossing index depends on the
// rounding), so one thread replays the sum in index order over chunks that
// the whole CTA stages into shared memory, stopping at the crossing.
constexpr int MP_CHUNK = 8192;

__global__ void __launch_bounds__(SM_THREADS) minp_kernel(SampleArgs a) {
	__shared__ float red[SM_NWARPS];
	__shared__ float chunk[MP_CHUNK];
	__shared__ int s_found;
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
	// (5)+(6)
	if (tid == 0) { s_found = -1; s_cum = 0.0f; }
	__syncthreads();
	int found = -1;
	for (int c0 = 0; c0 < a.V; c0 += MP_CHUNK) {
		for (int i = tid * 4; i < MP_CHUNK; i += SM_THREADS * 4) {
			float4 v = __ldcg(reinterpret_cast<const float4 *>(x + c0 + i));
			v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
			__stcg(reinterpret_cast<float4 *>(x + c0 + i), v);
			*reinterpret_cast<float4 *>(&chunk[i]) = v;
		}
		__syncthreads();
		if (tid == 0 && s_found < 0) {
			float cum = s_cum;
			int f = -1;
			for (int i = 0; i < MP_CHUNK; i++) {
				cum += chunk[i];
				if (cum >= randf) { f = c0 + i; break; }
			}
			s_cum = cum;
			s_found = f;
		}
		__syncthreads();
		found = s_found;
		// keep scaling the remaining chunks (the reference scales the whole row)
		// but stop replaying once the crossing is known
	}
	if (tid == 0) {
		emit_token(a, b, found < 0 ? 0 : found);
		a.randf_count[b] += 1;
	}
}

}  // namespace tg
