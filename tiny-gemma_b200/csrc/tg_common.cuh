// Shared device helpers for the sm_100a kernels of libtinygemma_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tg {

constexpr int WARP = 32;
constexpr float RMS_EPS = 1e-6f;  // reference ops.hpp:182 (default eps)

// ---------------------------------------------------------------- int8 -> fp32
// Exact conversion of the four int8 lanes of a 32-bit word without the
// (quarter-rate) integer-to-float unit: flip the sign bits so each byte holds
// w+128 in 0..255, drop that byte into the low mantissa byte of 2^23
// (0x4B000000) with one PRMT, and subtract 2^23+128. Every step is exact, so
// the result equals float(int8) bit for bit (reference linalg.hpp:8-37 does
// cvtepi8_epi32 + cvtepi32_ps).
__device__ __forceinline__ float i8_lane_to_f32(uint32_t biased_word, int lane) {
	uint32_t sel = 0x7650u + lane;
	return __uint_as_float(__byte_perm(biased_word, 0x4B000000u, sel)) - 8388736.0f;
}

__device__ __forceinline__ void i8x4_to_f32(uint32_t word, float (&f)[4]) {
	uint32_t b = word ^ 0x80808080u;
	f[0] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7650u)) - 8388736.0f;
	f[1] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7651u)) - 8388736.0f;
	f[2] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7652u)) - 8388736.0f;
	f[3] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7653u)) - 8388736.0f;
}

// streaming 128-bit load of weights: read once, keep out of L1
__device__ __forceinline__ int4 ld_stream_int4(const void *p) {
	int4 v;
	asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
	             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
	             : "l"(p));
	return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
	return v;
}

// Sum over a whole CTA in a fixed order (warp butterflies, then warps in index
// order by every thread) so that every CTA that reduces the same data gets the
// same bits. `red` is NWARPS floats of shared memory; safe to call repeatedly.
template <int NWARPS>
__device__ __forceinline__ float block_sum(float v, float *red) {
	v = warp_sum(v);
	__syncthreads();  // protect `red` from a previous use
	if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
	__syncthreads();
	float t = 0.0f;
#pragma unroll
	for (int w = 0; w < NWARPS; w++) t += red[w];
	return t;
}

// 1/sqrt(ms + eps) the IEEE way (reference ops.hpp:153 writes 1.0 / sqrt(x))
__device__ __forceinline__ float inv_rms(float sumsq, int dim) {
	float ms = sumsq / float(dim);
	return 1.0f / sqrtf(ms + RMS_EPS);
}

// lut::GeLUTable::lookup, reference ops.hpp:41-51
// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute may be
// scheduled while its predecessor in the stream still runs; it must call pdl_wait() before it touches
// anything a predecessor reads or writes (the call returns when every earlier grid has completed and its
// memory operations are visible). pdl_trigger() tells the scheduler that the NEXT kernel may be scheduled
// once every CTA of this grid has started. Without the attribute both are no-ops. What overlaps is launch
// latency, CTA scheduling and each kernel's own set-up (barrier initialisation, TMEM allocation, and in the
// GEMM the first weight tiles, which no earlier kernel produces).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct GeluLut {
	const float *table;
	float mn;
	float eps;
	int size;
	__device__ __forceinline__ float operator()(float x) const {
		float q = (x - mn) / eps;
		// x86 cvttss2si yields INT_MIN for NaN and out-of-range inputs, which the
		// reference then treats as a negative index
		if (!(q < 2147483648.0f) || q < -2147483648.0f) return 0.0f;
		int idx = int(q);
		if (idx < 0) return 0.0f;
		if (idx >= size) return x;
		return __ldg(table + idx);
	}
};

// sum over K-splits of p[sp * stride], added in ascending split order; the loads of up to eight
// splits are in flight together (missing splits contribute an exact + 0.0f). L2 = true reads around
// the L1 (ld.global.cg): for partial sums written by other CTAs of the SAME kernel.
template <bool L2 = false>
__device__ __forceinline__ float sum_splits(const float *p, size_t stride, int nsplit) {
	float v = 0.0f;
	for (int s0 = 0; s0 < nsplit; s0 += 8) {
		float a[8];
#pragma unroll
		for (int q = 0; q < 8; q++) {
			a[q] = 0.0f;
			if (s0 + q < nsplit) a[q] = L2 ? __ldcg(p + size_t(s0 + q) * stride) : p[size_t(s0 + q) * stride];
		}
#pragma unroll
		for (int q = 0; q < 8; q++) v += a[q];
	}
	return v;
}

}  // namespace tg
