// TEST INFRASTRUCTURE — the parity oracle. Not part of the product; nothing in
// the shipped library links, loads or calls this file.
//
// A plain scalar C++ restatement of tiny-gemma's int8 weight-only Gemma-3
// inference path (fattorib/tiny-gemma, csrc/include/*.hpp). Each function cites
// the reference file:line whose arithmetic it restates. It is written from the
// algorithm, with no SIMD intrinsics; where the reference's AVX2 code fixes an
// evaluation order (8-lane accumulators, horizontal-add trees, fused
// multiply-adds) the same order is kept with explicit std::fmaf so that results
// are bit-identical wherever IEEE arithmetic defines them.
//
// Known, documented differences from the compiled reference (Makefile:5 builds
// it with -ffast-math):
//   * 1/sqrt in RMSNorm: the reference compiles to the x86 RSQRTSS estimate +
//     one Newton step (CPU-vendor specific); here it is 1.0f / sqrtf(x).
//   * exp/pow/cos/sin/tanh: the reference links glibc's vector libm for some
//     loops; here scalar libm is used throughout.
// Compile with -O2 -mfma -ffp-contract=off (see oracle/build_oracle.py) so the
// compiler neither fuses nor splits what is written.
//
// Parity status: pinned. Checked against the compiled reference
// (oracle/_ref/libtgref.so) op by op and end to end, and against the
// reference's own NumPy-generated unit fixtures (tests/golden/).

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

namespace {

// ---------------------------------------------------------------- config
// reference config.hpp:7-48
struct Cfg {
	int D, I, L, V, n_pos, n_pos_local, hd, nh, nkv;
	float theta, theta_local;
	int pattern;
};
const Cfg CFG_270M{640, 2048, 18, 262144, 32768, 512, 256, 4, 1, 1000000.f, 10000.f, 6};
const Cfg CFG_1B{1152, 6912, 26, 262144, 32768, 512, 256, 4, 1, 1000000.f, 10000.f, 6};

bool get_cfg(const char *size, Cfg *out) {
	std::string s(size);
	if (s == "270m") {
		*out = CFG_270M;
		return true;
	}
	if (s == "1B") {
		*out = CFG_1B;
		return true;
	}
	return false;
}

thread_local std::string g_err;

// -------------------------------------------------------- lane reductions
// simd.hpp:16-32: four 8-lane accumulators -> (a+b)+(c+d) per lane, then
// hadd, hadd, low half + high half.
inline float reduce_4x8(const float acc[4][8]) {
	float t[8];
	for (int l = 0; l < 8; l++) t[l] = (acc[0][l] + acc[1][l]) + (acc[2][l] + acc[3][l]);
	float lo = (t[0] + t[1]) + (t[2] + t[3]);
	float hi = (t[4] + t[5]) + (t[6] + t[7]);
	return lo + hi;
}

// ----------------------------------------------------------------- matvec
// linalg.hpp:41-108 gemv::qgemv: for each k, y[n] += x[k]*W[k,n] (the fmadd
// into a zero accumulator followed by an add is a plain multiply then add),
// then y[n] *= scale[n]. y must be zero on entry (modules.hpp:137,206).
void qgemv(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	for (int k = 0; k < K; k++) {
		const float xk = x[k];
		const int8_t *wr = w + size_t(k) * N;
		for (int n = 0; n < N; n++) {
			float p = xk * float(wr[n]);
			y[n] = y[n] + p;
		}
	}
	for (int n = 0; n < N; n++) y[n] = y[n] * scales[n];
}

// linalg.hpp:112-174 gemv::qgemv_row_tile<K,N,T>: T rows at a time, an FMA
// chain from zero over the T rows, then added to y.
void qgemv_row_tile(float *y, const float *x, const int8_t *w, const float *scales, int K, int N, int T) {
	for (int k = 0; k < K; k += T) {
		for (int n = 0; n < N; n++) {
			float acc = 0.0f;
			for (int j = 0; j < T; j++) acc = std::fmaf(x[k + j], float(w[size_t(k + j) * N + n]), acc);
			y[n] = y[n] + acc;
		}
	}
	for (int n = 0; n < N; n++) y[n] = y[n] * scales[n];
}

// linalg.hpp:176-195 launch_qgemv: row tile 8 iff N == 6912
void linear_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	std::memset(y, 0, sizeof(float) * N);
	if (N == 6912)
		qgemv_row_tile(y, x, w, scales, K, N, 8);
	else
		qgemv(y, x, w, scales, K, N);
}

// linalg.hpp:197-204 launch_qgemv_logits: row tile 4
void lm_head_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	std::memset(y, 0, sizeof(float) * N);
	qgemv_row_tile(y, x, w, scales, K, N, 4);
}

// linalg.hpp:210-308 gemm::qgemmnn + microkernel: every output is one FMA
// chain over k = 0..K-1 from zero, then multiplied by scale[n].
void linear_prefill(float *c, const float *a, const int8_t *w, const float *scales, int M, int K, int N) {
	constexpr int MB = 8;
	std::vector<float> acc(size_t(MB) * N);
	for (int m0 = 0; m0 < M; m0 += MB) {
		int mb = std::min(MB, M - m0);
		std::fill(acc.begin(), acc.end(), 0.0f);
		for (int k = 0; k < K; k++) {
			const int8_t *wr = w + size_t(k) * N;
			for (int mi = 0; mi < mb; mi++) {
				const float av = a[size_t(m0 + mi) * K + k];
				float *ar = acc.data() + size_t(mi) * N;
				for (int n = 0; n < N; n++) ar[n] = std::fmaf(av, float(wr[n]), ar[n]);
			}
		}
		for (int mi = 0; mi < mb; mi++)
			for (int n = 0; n < N; n++) c[size_t(m0 + mi) * N + n] = acc[size_t(mi) * N + n] * scales[n];
	}
}

// ---------------------------------------------------------------- RMSNorm
// ops.hpp:126-180 rmsnorm_along_dim: sum of squares in 4 accumulators of 8
// lanes over 32-element chunks (the compiled reference contracts add(mul) to
// an FMA), mean, 1/sqrt(ms+eps), y = (x*r)*(w+1).
void rmsnorm_row(float *x, const float *w, int dim, float eps = 1e-6f) {
	float acc[4][8] = {};
	for (int d = 0; d < dim; d += 32)
		for (int j = 0; j < 4; j++)
			for (int l = 0; l < 8; l++) {
				float v = x[d + 8 * j + l];
				acc[j][l] = std::fmaf(v, v, acc[j][l]);
			}
	float ms = reduce_4x8(acc) / float(dim);
	float r = 1.0f / std::sqrt(ms + eps);
	for (int d = 0; d < dim; d++) x[d] = (x[d] * r) * (w[d] + 1.0f);
}

// ------------------------------------------------------------- GeLU table
// ops.hpp:16-51: tanh-GeLU evaluated in double (the literals 0.5 and 3.0 are
// double), step table with no interpolation.
struct GeluTable {
	float mn, mx, eps;
	int size;
	std::vector<float> t;
	void build(float mn_, float mx_, int size_) {
		mn = mn_;
		mx = mx_;
		size = size_;
		eps = float(mx - mn) / float(size);
		t.resize(size);
		for (int i = 0; i < size; i++) {
			float a = float(mn) + i * eps;
			const float c0 = 0.7978845608f, c1 = 0.044715f;
			double inner = double(c0) * (double(a) + double(c1) * std::pow(double(a), 3.0));
			t[i] = float((0.5 * double(a)) * (1.0 + std::tanh(inner)));
		}
	}
	inline float lookup(float x) const {
		int idx = int((x - mn) / eps);
		if (idx < 0) return 0.0f;
		if (idx >= size) return x;
		return t[idx];
	}
};

// ------------------------------------------------------------------- RoPE
// decode.hpp:176-201 pre_compute_freqs: float powf, reciprocal in double,
// float cos/sin of float(p)*freq, written to both halves.
void rope_tables(float theta, int max_pos, int dhead, float *cosT, float *sinT) {
	int half = dhead / 2;
	std::vector<float> freqs(half);
	for (int i = 0; i < half; i++) {
		float denom = std::pow(theta, float(2 * i) / dhead);
		freqs[i] = float(1.0 / denom);
	}
	for (int p = 0; p < max_pos; p++)
		for (int d = 0; d < half; d++) {
			float outer = p * freqs[d];
			float c = std::cos(outer), s = std::sin(outer);
			cosT[size_t(p) * dhead + d] = c;
			cosT[size_t(p) * dhead + d + half] = c;
			sinT[size_t(p) * dhead + d] = s;
			sinT[size_t(p) * dhead + d + half] = s;
		}
}

// decode.hpp:136-174,203-211 apply_rotary_emb on one head vector at position
// pos: y = cos*x + rotate_half(x)*sin with rotate_half = [-x2, x1]. The
// reference's scalar loop is compiled with fast-math contraction:
// fma(rot, sin, cos*x).
void rope_apply(float *x, const float *cosT, const float *sinT, int pos, int dhead) {
	int half = dhead / 2;
	float rot[512];
	for (int i = 0; i < half; i++) {
		rot[i] = -1.0f * x[i + half];
		rot[i + half] = x[i];
	}
	const float *c = cosT + size_t(pos) * dhead, *s = sinT + size_t(pos) * dhead;
	for (int d = 0; d < dhead; d++) x[d] = std::fmaf(rot[d], s[d], c[d] * x[d]);
}

// --------------------------------------------------------------- KV cache
// decode.hpp:14-105
struct KV {
	std::vector<float> k, v;  // [max_pos, hd]
	int position_ptr = 0, buffer_ptr = 0, max_pos = 0, hd = 0;
	bool is_sw = false;
	void init(const Cfg &c, bool sw) {
		is_sw = sw;
		max_pos = sw ? c.n_pos_local : c.n_pos;
		hd = c.hd;
		k.assign(size_t(max_pos) * hd, 0.0f);
		v.assign(size_t(max_pos) * hd, 0.0f);
		position_ptr = buffer_ptr = 0;
	}
	int valid_pos() const { return max_pos > position_ptr ? position_ptr : max_pos; }
	// decode.hpp:49-70
	void update_single(const float *key, const float *val) {
		size_t off = size_t(buffer_ptr % max_pos) * hd;
		std::memcpy(&k[off], key, sizeof(float) * hd);
		std::memcpy(&v[off], val, sizeof(float) * hd);
		buffer_ptr += 1;
		position_ptr += 1;
	}
	// decode.hpp:72-105: needs an empty cache; keeps the prompt tail
	bool update_prefill(const float *keys, const float *vals, int S) {
		if (position_ptr != 0 || buffer_ptr != 0) return false;
		int start = (S >= max_pos) ? (S - max_pos) : 0;
		for (int s = start, c = 0; s < S; s++, c++) {
			std::memcpy(&k[size_t(c) * hd], keys + size_t(s) * hd, sizeof(float) * hd);
			std::memcpy(&v[size_t(c) * hd], vals + size_t(s) * hd, sizeof(float) * hd);
		}
		buffer_ptr += (start > 0) ? max_pos : S;
		position_ptr += S;
		return true;
	}
};

// -------------------------------------------------------------- attention
// 256-long dot product in the reference's lane structure (ops.hpp:299-314):
// four 8-lane FMA accumulators over 32-element chunks, reduced with
// reduce_horizontalx4.
inline float dot_lanes(const float *a, const float *b, int dim) {
	float acc[4][8] = {};
	for (int d = 0; d < dim; d += 32)
		for (int j = 0; j < 4; j++)
			for (int l = 0; l < 8; l++) acc[j][l] = std::fmaf(a[d + 8 * j + l], b[d + 8 * j + l], acc[j][l]);
	return reduce_4x8(acc);
}

// ops.hpp:224-370 attention_decode: q [nh, hd] (one query), cache slots
// 0..valid_pos-1 in buffer order, output renormalised at every key.
void attention_decode(float *o, const float *q, const KV &kv, int nh, int hd) {
	const float scale = float(1.0 / std::sqrt(float(hd)));
	std::vector<float> qs(size_t(nh) * hd), ot(size_t(nh) * hd, 0.0f);
	std::vector<float> ms(nh, -INFINITY), ls(nh, 0.0f);
	for (int i = 0; i < nh * hd; i++) qs[i] = q[i] * scale;
	int seq = kv.valid_pos();
	for (int i = 0; i < seq; i++) {
		const float *kt = &kv.k[size_t(i) * hd], *vt = &kv.v[size_t(i) * hd];
		for (int h = 0; h < nh; h++) {
			float s = dot_lanes(&qs[size_t(h) * hd], kt, hd);
			float m = std::fmax(ms[h], s);
			float corr = std::exp(ms[h] - m);
			float update = std::exp(s - m);
			float l_new = (corr * ls[h]) + update;
			float il_new = float(1.0 / l_new);
			float *oh = &ot[size_t(h) * hd];
			for (int d = 0; d < hd; d++) {
				float t = ls[h] * oh[d];
				t = corr * t;
				t = std::fmaf(update, vt[d], t);
				oh[d] = t * il_new;
			}
			ms[h] = m;
			ls[h] = l_new;
		}
	}
	std::memcpy(o, ot.data(), sizeof(float) * nh * hd);
}

// ops.hpp:377-526 attention_prefill: q,o [nh, S, hd]; k,v [S, hd]; causal, and
// on sliding-window layers keys qs-sw_context..qs (sw_context+1 keys, :437-443);
// lazy softmax (Rabe & Staats) with the branch on s > m*.
void attention_prefill(float *o, const float *q, const float *k, const float *v, int nh, int S, int hd, bool is_sw,
                       int sw_context) {
	const float scale = float(1.0 / std::sqrt(float(hd)));
	std::vector<float> acc(hd);
	for (int h = 0; h < nh; h++)
		for (int qi = 0; qi < S; qi++) {
			const float *qt = q + (size_t(h) * S + qi) * hd;
			std::fill(acc.begin(), acc.end(), 0.0f);
			float s_star = 0.0f, m_star = -INFINITY;
			int k0 = 0;
			if (is_sw) k0 = (qi >= sw_context) ? qi - sw_context : 0;
			for (int ki = k0; ki <= qi; ki++) {
				const float *kt = k + size_t(ki) * hd, *vt = v + size_t(ki) * hd;
				float s = dot_lanes(qt, kt, hd);
				s = s * scale;
				float m = std::fmax(m_star, s);
				float corr, update;
				if (s > m_star) {
					corr = std::exp(m_star - s);
					update = 1.0f;
				} else {
					corr = 1.0f;
					update = std::exp(s - m_star);
				}
				for (int d = 0; d < hd; d++) acc[d] = std::fmaf(vt[d], update, acc[d] * corr);
				s_star = (s_star * corr) + update;
				m_star = m;
			}
			const float inv = float(1.0 / s_star);
			float *ot = o + (size_t(h) * S + qi) * hd;
			for (int d = 0; d < hd; d++) ot[d] = acc[d] * inv;
		}
}

// ----------------------------------------------------------------- layers
struct QW {
	const int8_t *q = nullptr;
	const float *s = nullptr;
	int K = 0, N = 0;
};
struct AttnW {
	QW Q, K, V, O;
	const float *rmsq, *rmsk, *pre, *post;
	bool is_sw;
};
struct MlpW {
	QW U, G, Dn;
	const float *pre, *post;
};

void linear(float *y, const float *x, const QW &w, int S) {
	if (S == 1)
		linear_decode(y, x, w.q, w.s, w.K, w.N);
	else
		linear_prefill(y, x, w.q, w.s, S, w.K, w.N);
}

// modules.hpp:89-169 attention (both branches); x [S, D] in place.
bool module_attention(float *x, int S, const Cfg &c, const AttnW &w, KV &kv, const float *cosT, const float *sinT) {
	const int D = c.D, hd = c.hd, nh = c.nh, qd = nh * hd;
	std::vector<float> xr(x, x + size_t(S) * D);
	for (int s = 0; s < S; s++) rmsnorm_row(x + size_t(s) * D, w.pre, D);
	std::vector<float> xq(size_t(S) * qd), xk(size_t(S) * hd), xv(size_t(S) * hd);
	linear(xq.data(), x, w.Q, S);
	linear(xk.data(), x, w.K, S);
	linear(xv.data(), x, w.V, S);
	// split_rearrange [S, nh*hd] -> [nh, S, hd] (ops.hpp:670-706)
	std::vector<float> qs(size_t(S) * qd), os(size_t(S) * qd);
	for (int s = 0; s < S; s++)
		for (int h = 0; h < nh; h++)
			std::memcpy(&qs[(size_t(h) * S + s) * hd], &xq[size_t(s) * qd + size_t(h) * hd], sizeof(float) * hd);
	int pos0 = (S > 1) ? 0 : kv.position_ptr;
	for (int h = 0; h < nh; h++)
		for (int s = 0; s < S; s++) {
			float *v = &qs[(size_t(h) * S + s) * hd];
			rmsnorm_row(v, w.rmsq, hd);
		}
	for (int s = 0; s < S; s++) rmsnorm_row(&xk[size_t(s) * hd], w.rmsk, hd);
	for (int h = 0; h < nh; h++)
		for (int s = 0; s < S; s++) rope_apply(&qs[(size_t(h) * S + s) * hd], cosT, sinT, pos0 + s, hd);
	for (int s = 0; s < S; s++) rope_apply(&xk[size_t(s) * hd], cosT, sinT, pos0 + s, hd);
	if (S > 1) {
		if (!kv.update_prefill(xk.data(), xv.data(), S)) return false;
		attention_prefill(os.data(), qs.data(), xk.data(), xv.data(), nh, S, hd, kv.is_sw, kv.max_pos);
	} else {
		kv.update_single(xk.data(), xv.data());
		attention_decode(os.data(), qs.data(), kv, nh, hd);
	}
	// fuse_rearrange [nh, S, hd] -> [S, nh*hd] (ops.hpp:708-742)
	std::vector<float> xo(size_t(S) * qd);
	for (int h = 0; h < nh; h++)
		for (int s = 0; s < S; s++)
			std::memcpy(&xo[size_t(s) * qd + size_t(h) * hd], &os[(size_t(h) * S + s) * hd], sizeof(float) * hd);
	linear(x, xo.data(), w.O, S);
	for (int s = 0; s < S; s++) rmsnorm_row(x + size_t(s) * D, w.post, D);
	for (size_t i = 0; i < size_t(S) * D; i++) x[i] = x[i] + xr[i];
	return true;
}

// modules.hpp:171-221 mlp; x [S, D] in place.
void module_mlp(float *x, int S, const Cfg &c, const MlpW &w, const GeluTable &table) {
	const int D = c.D, I = w.U.N;
	std::vector<float> xr(x, x + size_t(S) * D);
	for (int s = 0; s < S; s++) rmsnorm_row(x + size_t(s) * D, w.pre, D);
	std::vector<float> up(size_t(S) * I), gate(size_t(S) * I);
	linear(up.data(), x, w.U, S);
	linear(gate.data(), x, w.G, S);
	for (size_t i = 0; i < gate.size(); i++) gate[i] = table.lookup(gate[i]) * up[i];
	linear(x, gate.data(), w.Dn, S);
	for (int s = 0; s < S; s++) rmsnorm_row(x + size_t(s) * D, w.post, D);
	for (size_t i = 0; i < size_t(S) * D; i++) x[i] = x[i] + xr[i];
}

// modules.hpp:223-247 lm_head: final norm on the last position, row-tile-4 matvec
void module_lm_head(float *logits, const float *x, int S, int D, const QW &w, const float *rmsw) {
	std::vector<float> t(x + size_t(S - 1) * D, x + size_t(S) * D);
	rmsnorm_row(t.data(), rmsw, D);
	lm_head_decode(logits, t.data(), w.q, w.s, w.K, w.N);
}

// ops.hpp:529-616 embedding: x[d] = scale[d] * (sqrt(D) * float(wte[tok,d]))
void embedding(float *x, int tok, const int8_t *wte, const float *scales, int D) {
	const float sc = float(std::sqrt(double(D)));
	for (int d = 0; d < D; d++) x[d] = scales[d] * (sc * float(wte[size_t(tok) * D + d]));
}

// ------------------------------------------------------------------ model
struct Model {
	Cfg c;
	std::vector<uint8_t> blob;
	const int8_t *wte;
	const float *wte_s, *final_norm;
	std::vector<AttnW> attn;
	std::vector<MlpW> mlp;
	QW lm_head;
};

size_t model_bytes(const Cfg &c) {
	size_t qd = size_t(c.nh) * c.hd, kd = size_t(c.nkv) * c.hd, D = c.D, I = c.I, V = c.V;
	size_t per_layer = D * qd + 4 * qd + 2 * (D * kd + 4 * kd) + qd * D + 4 * D + 2 * 4 * c.hd + 2 * 4 * D +
	                   2 * (D * I + 4 * I) + I * D + 4 * D + 2 * 4 * D;
	return V * D + 4 * D + 4 * D + c.L * per_layer + D * V + 4 * V;
}

// transformer.hpp:99-165 read_weights order
void bind_model(Model *m) {
	const Cfg &c = m->c;
	const uint8_t *p = m->blob.data();
	auto take = [&](size_t n) {
		const uint8_t *r = p;
		p += n;
		return r;
	};
	auto takeq = [&](int K, int N) {
		QW w;
		w.K = K;
		w.N = N;
		w.q = reinterpret_cast<const int8_t *>(take(size_t(K) * N));
		w.s = reinterpret_cast<const float *>(take(4 * size_t(N)));
		return w;
	};
	auto takef = [&](int n) { return reinterpret_cast<const float *>(take(4 * size_t(n))); };
	int qd = c.nh * c.hd, kd = c.nkv * c.hd;
	m->wte = reinterpret_cast<const int8_t *>(take(size_t(c.V) * c.D));
	m->wte_s = takef(c.D);
	m->final_norm = takef(c.D);
	m->attn.resize(c.L);
	m->mlp.resize(c.L);
	for (int l = 0; l < c.L; l++) {
		AttnW &a = m->attn[l];
		a.Q = takeq(c.D, qd);
		a.K = takeq(c.D, kd);
		a.V = takeq(c.D, kd);
		a.O = takeq(qd, c.D);
		a.rmsq = takef(c.hd);
		a.rmsk = takef(c.hd);
		a.pre = takef(c.D);
		a.post = takef(c.D);
		a.is_sw = (l % c.pattern) != (c.pattern - 1);
		MlpW &w = m->mlp[l];
		w.U = takeq(c.D, c.I);
		w.G = takeq(c.D, c.I);
		w.Dn = takeq(c.I, c.D);
		w.pre = takef(c.D);
		w.post = takef(c.D);
	}
	m->lm_head = takeq(c.D, c.V);
}

struct State {
	Model *m;
	std::vector<KV> kv;
	std::vector<float> cos_g, sin_g, cos_l, sin_l;
	GeluTable table;
	std::vector<float> hidden;
};

// transformer.hpp:49-97 forward_prefill / forward_decode (S > 1 / S == 1)
bool forward(State *s, const int *ids, int S, float *logits) {
	const Cfg &c = s->m->c;
	std::vector<float> x(size_t(S) * c.D);
	for (int i = 0; i < S; i++) embedding(&x[size_t(i) * c.D], ids[i], s->m->wte, s->m->wte_s, c.D);
	for (int l = 0; l < c.L; l++) {
		const AttnW &a = s->m->attn[l];
		const float *ct = a.is_sw ? s->cos_l.data() : s->cos_g.data();
		const float *st = a.is_sw ? s->sin_l.data() : s->sin_g.data();
		if (!module_attention(x.data(), S, c, a, s->kv[l], ct, st)) {
			g_err = "update_prefill on a non-empty cache";
			return false;
		}
		module_mlp(x.data(), S, c, s->m->mlp[l], s->table);
	}
	s->hidden.assign(x.begin() + size_t(S - 1) * c.D, x.end());
	rmsnorm_row(s->hidden.data(), s->m->final_norm, c.D);
	lm_head_decode(logits, s->hidden.data(), s->m->lm_head.q, s->m->lm_head.s, c.D, c.V);
	return true;
}

// ops.hpp:744-760
int argmax_logits(const float *x, int n) {
	float best = -INFINITY;
	int arg = -1;
	for (int i = 0; i < n; i++)
		if (x[i] > best) {
			arg = i;
			best = x[i];
		}
	return arg;
}

// ops.hpp:762-859. Mutates x into the reference's "probabilities" (tokens
// below the cut keep their mass; only the denominator is masked).
int minp_logits(float *x, int n, float minp, float temp, float randf) {
	for (int i = 0; i < n; i++) x[i] /= temp;
	float rowmax = -INFINITY;
	for (int i = 0; i < n; i++) rowmax = std::fmax(rowmax, x[i]);
	float maxp = -INFINITY;
	for (int i = 0; i < n; i++) {
		x[i] = std::exp(x[i] - rowmax);
		if (x[i] > maxp) maxp = x[i];
	}
	float cut = minp * maxp;
	float acc[4][8] = {};
	for (int i = 0; i < n; i += 32)
		for (int j = 0; j < 4; j++)
			for (int l = 0; l < 8; l++) {
				float p = x[i + 8 * j + l];
				acc[j][l] += (p < cut) ? 0.0f : p;
			}
	float denom = reduce_4x8(acc);
	float inv = float(1.0 / denom);
	for (int i = 0; i < n; i++) x[i] = x[i] * inv;
	float cum = 0.0f;
	int index = 0;
	for (int i = 0; i < n; i++) {
		cum += x[i];
		if (cum >= randf) {
			index = i;
			break;
		}
	}
	return index;
}

}  // namespace

// =================================================================== C ABI
extern "C" {

const char *orc_last_error() { return g_err.c_str(); }
const char *orc_kind() { return "port"; }

void *orc_model_create(const char *size) {
	Cfg c;
	if (!get_cfg(size, &c)) {
		g_err = "unknown model size";
		return nullptr;
	}
	Model *m = new Model();
	m->c = c;
	return m;
}
void orc_model_free(void *m) { delete static_cast<Model *>(m); }

int orc_model_load(void *mp, const char *path) {
	Model *m = static_cast<Model *>(mp);
	FILE *f = std::fopen(path, "rb");
	if (!f) {
		g_err = "Could not open file.";
		return 1;
	}
	size_t want = model_bytes(m->c);
	m->blob.resize(want);
	size_t got = std::fread(m->blob.data(), 1, want, f);
	std::fclose(f);
	if (got != want) {
		g_err = "short read";
		return 2;
	}
	bind_model(m);
	return 0;
}

void *orc_state_create(void *mp, int gelu_size) {
	Model *m = static_cast<Model *>(mp);
	State *s = new State();
	s->m = m;
	const Cfg &c = m->c;
	s->kv.resize(c.L);
	for (int l = 0; l < c.L; l++) s->kv[l].init(c, (l % c.pattern) != (c.pattern - 1));
	size_t n = size_t(c.n_pos) * c.hd;
	s->cos_g.resize(n);
	s->sin_g.resize(n);
	s->cos_l.resize(n);
	s->sin_l.resize(n);
	rope_tables(c.theta, c.n_pos, c.hd, s->cos_g.data(), s->sin_g.data());
	rope_tables(c.theta_local, c.n_pos, c.hd, s->cos_l.data(), s->sin_l.data());
	s->table.build(-4.0f, 4.0f, gelu_size);
	return s;
}
void orc_state_free(void *s) { delete static_cast<State *>(s); }

// replace the state's tables (e.g. with the compiled reference's own)
int orc_state_set_tables(void *sp, const float *cos_g, const float *sin_g, const float *cos_l, const float *sin_l,
                         const float *gelu) {
	State *s = static_cast<State *>(sp);
	size_t n = s->cos_g.size();
	if (cos_g) std::memcpy(s->cos_g.data(), cos_g, 4 * n);
	if (sin_g) std::memcpy(s->sin_g.data(), sin_g, 4 * n);
	if (cos_l) std::memcpy(s->cos_l.data(), cos_l, 4 * n);
	if (sin_l) std::memcpy(s->sin_l.data(), sin_l, 4 * n);
	if (gelu) std::memcpy(s->table.t.data(), gelu, 4 * size_t(s->table.size));
	return 0;
}

int orc_state_tables(void *sp, float *cos_g, float *sin_g, float *cos_l, float *sin_l, float *gelu) {
	State *s = static_cast<State *>(sp);
	size_t n = s->cos_g.size();
	if (cos_g) std::memcpy(cos_g, s->cos_g.data(), 4 * n);
	if (sin_g) std::memcpy(sin_g, s->sin_g.data(), 4 * n);
	if (cos_l) std::memcpy(cos_l, s->cos_l.data(), 4 * n);
	if (sin_l) std::memcpy(sin_l, s->sin_l.data(), 4 * n);
	if (gelu) std::memcpy(gelu, s->table.t.data(), 4 * size_t(s->table.size));
	return 0;
}

int orc_prefill(void *sp, const int *ids, int n, float *logits) {
	State *s = static_cast<State *>(sp);
	std::vector<float> tmp;
	if (!logits) {
		tmp.resize(s->m->c.V);
		logits = tmp.data();
	}
	return forward(s, ids, n, logits) ? 0 : 1;
}

int orc_decode(void *sp, int tok, float *logits) {
	State *s = static_cast<State *>(sp);
	std::vector<float> tmp;
	if (!logits) {
		tmp.resize(s->m->c.V);
		logits = tmp.data();
	}
	return forward(s, &tok, 1, logits) ? 0 : 1;
}

int orc_decode_loop(void *sp, int first_tok, int n_steps, float minp, float temp, const float *randf, int *toks_out) {
	State *s = static_cast<State *>(sp);
	std::vector<float> logits(s->m->c.V);
	int tok = first_tok;
	for (int i = 0; i < n_steps; i++) {
		if (!forward(s, &tok, 1, logits.data())) return 1;
		tok = randf ? minp_logits(logits.data(), s->m->c.V, minp, temp, randf[i]) : argmax_logits(logits.data(), s->m->c.V);
		toks_out[i] = tok;
	}
	return 0;
}

int orc_kv_info(void *sp, int layer, int *position_ptr, int *buffer_ptr, int *max_pos) {
	State *s = static_cast<State *>(sp);
	*position_ptr = s->kv[layer].position_ptr;
	*buffer_ptr = s->kv[layer].buffer_ptr;
	*max_pos = s->kv[layer].max_pos;
	return 0;
}

int orc_kv_read(void *sp, int layer, int slot0, int nslots, float *k_out, float *v_out) {
	State *s = static_cast<State *>(sp);
	KV &kv = s->kv[layer];
	std::memcpy(k_out, &kv.k[size_t(slot0) * kv.hd], sizeof(float) * kv.hd * nslots);
	std::memcpy(v_out, &kv.v[size_t(slot0) * kv.hd], sizeof(float) * kv.hd * nslots);
	return 0;
}

int orc_hidden_read(void *sp, float *out) {
	State *s = static_cast<State *>(sp);
	std::memcpy(out, s->hidden.data(), sizeof(float) * s->hidden.size());
	return 0;
}

int orc_argmax_logits(const float *logits, int n) { return argmax_logits(logits, n); }
int orc_minp_logits(float *logits, int n, float minp, float temp, float randf) {
	return minp_logits(logits, n, minp, temp, randf);
}

int orc_linear_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	linear_decode(y, x, w, scales, K, N);
	return 0;
}
int orc_lm_head_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	lm_head_decode(y, x, w, scales, K, N);
	return 0;
}
int orc_linear_prefill(float *c, const float *a, const int8_t *w, const float *scales, int M, int K, int N) {
	linear_prefill(c, a, w, scales, M, K, N);
	return 0;
}

int orc_time_linear(const float *x, const int8_t *w, const float *scales, int M, int K, int N, int reps, double *secs) {
	std::vector<float> y(size_t(M) * N);
	auto t0 = std::chrono::high_resolution_clock::now();
	for (int r = 0; r < reps; r++) {
		if (M == 1) {
			if (N == 262144)
				lm_head_decode(y.data(), x, w, scales, K, N);
			else
				linear_decode(y.data(), x, w, scales, K, N);
		} else
			linear_prefill(y.data(), x, w, scales, M, K, N);
	}
	auto t1 = std::chrono::high_resolution_clock::now();
	*secs = (t1 - t0).count() / 1e9;
	return 0;
}

int orc_rmsnorm(float *x, const float *w, int rows, int dim) {
	for (int r = 0; r < rows; r++) rmsnorm_row(x + size_t(r) * dim, w, dim);
	return 0;
}

int orc_rope_tables(const char *size, int is_local, float *cos_out, float *sin_out) {
	Cfg c;
	if (!get_cfg(size, &c)) return 1;
	rope_tables(is_local ? c.theta_local : c.theta, c.n_pos, c.hd, cos_out, sin_out);
	return 0;
}

int orc_gelu_table(float mn, float mx, int size, float *out) {
	GeluTable t;
	t.build(mn, mx, size);
	std::memcpy(out, t.t.data(), 4 * size_t(size));
	return 0;
}

int orc_module_mlp(float *x, int S, int D, int I, const int8_t *uw, const float *us, const int8_t *gw, const float *gs,
                   const int8_t *dw, const float *ds, const float *pre, const float *post, int gelu_size) {
	Cfg c = (D == 640) ? CFG_270M : CFG_1B;
	MlpW w;
	w.U = QW{uw, us, D, I};
	w.G = QW{gw, gs, D, I};
	w.Dn = QW{dw, ds, I, D};
	w.pre = pre;
	w.post = post;
	GeluTable t;
	t.build(-4.0f, 4.0f, gelu_size);
	module_mlp(x, S, c, w, t);
	return 0;
}

int orc_module_attention(float *x, int S, int D, int is_sw, const int8_t *qw, const float *qs, const int8_t *kw,
                         const float *ks, const int8_t *vw, const float *vs, const int8_t *ow, const float *os,
                         const float *rmsq, const float *rmsk, const float *pre, const float *post, int n_cached,
                         const float *k_cache, const float *v_cache) {
	Cfg c = (D == 640) ? CFG_270M : CFG_1B;
	int qd = c.nh * c.hd, kd = c.nkv * c.hd;
	AttnW w;
	w.Q = QW{qw, qs, D, qd};
	w.K = QW{kw, ks, D, kd};
	w.V = QW{vw, vs, D, kd};
	w.O = QW{ow, os, qd, D};
	w.rmsq = rmsq;
	w.rmsk = rmsk;
	w.pre = pre;
	w.post = post;
	w.is_sw = is_sw != 0;
	KV kv;
	kv.init(c, is_sw != 0);
	if (S == 1 && n_cached > 0) {
		std::memcpy(kv.k.data(), k_cache, sizeof(float) * size_t(n_cached) * c.hd);
		std::memcpy(kv.v.data(), v_cache, sizeof(float) * size_t(n_cached) * c.hd);
		kv.position_ptr = kv.buffer_ptr = n_cached;
	}
	size_t n = size_t(c.n_pos) * c.hd;
	std::vector<float> ct(n), st(n);
	rope_tables(is_sw ? c.theta_local : c.theta, c.n_pos, c.hd, ct.data(), st.data());
	return module_attention(x, S, c, w, kv, ct.data(), st.data()) ? 0 : 1;
}

int orc_module_lm_head(float *logits, const float *x, int S, int D, const int8_t *w, const float *scales,
                       const float *rmsw) {
	QW q{w, scales, D, 262144};
	module_lm_head(logits, x, S, D, q, rmsw);
	return 0;
}

// std::mt19937 + uniform_real_distribution<float>(0,1), the generator the
// reference's generate() draws randf from (transformer.hpp:170-172)
int orc_mt19937_uniforms(unsigned seed, int n, float *out) {
	std::mt19937 gen(seed);
	std::uniform_real_distribution<float> unif(0.0, 1.0);
	for (int i = 0; i < n; i++) out[i] = unif(gen);
	return 0;
}

}  // extern "C"
