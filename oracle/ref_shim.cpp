// TEST INFRASTRUCTURE — not part of the product.
//
// Thin extern "C" shim around the UNMODIFIED tiny-gemma reference headers
// (csrc/include/*.hpp of fattorib/tiny-gemma). The headers are included from
// where they lie (the include path is given on the g++ command line by
// oracle/build_oracle.py); no reference source is copied into this repo.
// The resulting library, oracle/_ref/libtgref.so, is the strongest form of
// the parity oracle: the reference's own AVX2 code compiled with the
// reference's own flags (Makefile:5), callable from the Python tests and from
// bench.py's cpu_baseline / --impl reference legs.
//
// Every entry point mirrors one function of oracle/tg_oracle.cpp (prefix orc_)
// so that the same Python wrapper drives either library.
//
// The reference keeps large arrays on the stack (gemm::qgemmnn packs 256 x K
// floats there, csrc/include/linalg.hpp:258), so every call runs on a
// dedicated thread with a 512 MiB stack. That thread also sets FTZ/DAZ the way
// an executable linked with -ffast-math does at start-up.

#include <pthread.h>
#include <xmmintrin.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "config.hpp"
#include "transformer.hpp"

namespace {

struct Job {
	std::function<void(void)> fn;
	std::string err;
};

void *job_main(void *p) {
	Job *j = static_cast<Job *>(p);
	_mm_setcsr(_mm_getcsr() | 0x8040);  // FTZ | DAZ, as crtfastmath.o would
	try {
		j->fn();
	} catch (const std::exception &e) {
		j->err = e.what();
	}
	return nullptr;
}

thread_local std::string g_err;

int run_big_stack(std::function<void(void)> fn) {
	Job j{std::move(fn), {}};
	pthread_attr_t attr;
	pthread_attr_init(&attr);
	pthread_attr_setstacksize(&attr, size_t(512) << 20);
	pthread_t th;
	if (pthread_create(&th, &attr, job_main, &j) != 0) {
		g_err = "pthread_create failed";
		return 1;
	}
	pthread_join(th, nullptr);
	pthread_attr_destroy(&attr);
	if (!j.err.empty()) {
		g_err = j.err;
		return 1;
	}
	return 0;
}

struct RefModel {
	config::Config cfg;
	gemma::Transformer t;
	explicit RefModel(const config::Config &c) : cfg(c), t(c) {}
};

struct RefState {
	RefModel *m;
	decode::RoPE rope;
	decode::RoPE rope_sw;
	lut::GeLUTable table;
	decode::DecodeState d;
	tensor::activation o;
	RefState(RefModel *m, int gelu_size)
	    : m(m), rope(&m->cfg, false), rope_sw(&m->cfg, true), table(-4.0, 4.0, gelu_size), d(1, &m->cfg), o(1, 1, m->cfg.n_vocab) {}
};

tensor::QuantArray borrow_weight(const int8_t *w, const float *scales, int K, int N) {
	tensor::QuantArray q(K, N, true);
	std::memcpy(q.data.get(), w, size_t(K) * N);
	std::memcpy(q.scales.get(), scales, sizeof(float) * N);
	return q;
}

tensor::FloatArray make_f(const float *w, int n) {
	tensor::FloatArray f(n);
	std::memcpy(f.data.get(), w, sizeof(float) * n);
	return f;
}

}  // namespace

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }
const char *ref_kind() { return "reference"; }

void *ref_model_create(const char *size) {
	auto it = config::CONFIG_MAP.find(size);
	if (it == config::CONFIG_MAP.end()) {
		g_err = "unknown model size";
		return nullptr;
	}
	return new RefModel(it->second);
}

void ref_model_free(void *m) { delete static_cast<RefModel *>(m); }

int ref_model_load(void *m, const char *path) {
	RefModel *rm = static_cast<RefModel *>(m);
	return run_big_stack([&] { gemma::read_weights(&rm->t, path); });
}

void *ref_state_create(void *m, int gelu_size) {
	RefState *s = nullptr;
	int rc = run_big_stack([&] { s = new RefState(static_cast<RefModel *>(m), gelu_size); });
	return rc == 0 ? s : nullptr;
}

void ref_state_free(void *s) { delete static_cast<RefState *>(s); }

// transformer.hpp:49 forward_prefill; logits [n_vocab] copied to `logits` if non-null
int ref_prefill(void *sp, const int *ids, int n, float *logits) {
	RefState *s = static_cast<RefState *>(sp);
	return run_big_stack([&] {
		auto td = tensor::make_unique_aligned<int>(n);
		for (int i = 0; i < n; i++) td[i] = ids[i];
		tensor::tokens toks(td, 1, n);
		gemma::forward_prefill(&s->o, &toks, &s->m->t, &s->d, &s->rope, &s->rope_sw, &s->table);
		if (logits) std::memcpy(logits, s->o.data.get(), sizeof(float) * s->m->cfg.n_vocab);
	});
}

// transformer.hpp:75 forward_decode
int ref_decode(void *sp, int tok, float *logits) {
	RefState *s = static_cast<RefState *>(sp);
	return run_big_stack([&] {
		tensor::tokens toks(1, 1);
		toks.data[0] = tok;
		gemma::forward_decode(&s->o, &toks, &s->m->t, &s->d, &s->rope, &s->rope_sw, 0, &s->table);
		if (logits) std::memcpy(logits, s->o.data.get(), sizeof(float) * s->m->cfg.n_vocab);
	});
}

// Runs `n_steps` of decode + sampler entirely inside the library (one thread
// start for the whole loop) — the CPU-baseline timing loop. `randf` may be
// null (greedy, ops.hpp:744) or hold n_steps uniforms (min-p, ops.hpp:762).
// tok_io: in = first token to feed, out[n_steps] = sampled tokens.
int ref_decode_loop(void *sp, int first_tok, int n_steps, float minp, float temp, const float *randf, int *toks_out) {
	RefState *s = static_cast<RefState *>(sp);
	return run_big_stack([&] {
		tensor::tokens toks(1, 1);
		toks.data[0] = first_tok;
		for (int i = 0; i < n_steps; i++) {
			gemma::forward_decode(&s->o, &toks, &s->m->t, &s->d, &s->rope, &s->rope_sw, 0, &s->table);
			if (randf)
				ops::minp_logits(&toks, &s->o, minp, temp, randf[i]);
			else
				ops::argmax_logits(&toks, &s->o);
			toks_out[i] = toks.data[0];
		}
	});
}

// state introspection for parity checks
int ref_kv_info(void *sp, int layer, int *position_ptr, int *buffer_ptr, int *max_pos) {
	RefState *s = static_cast<RefState *>(sp);
	decode::KVCache &kv = s->d.kvcache[layer];
	*position_ptr = kv.position_ptr;
	*buffer_ptr = kv.buffer_ptr;
	*max_pos = kv.max_pos;
	return 0;
}

int ref_kv_read(void *sp, int layer, int slot0, int nslots, float *k_out, float *v_out) {
	RefState *s = static_cast<RefState *>(sp);
	decode::KVCache &kv = s->d.kvcache[layer];
	size_t hd = kv.head_dim;
	std::memcpy(k_out, kv.keys.data.get() + slot0 * hd, sizeof(float) * hd * nslots);
	std::memcpy(v_out, kv.values.data.get() + slot0 * hd, sizeof(float) * hd * nslots);
	return 0;
}

// final hidden state after the last forward_decode (already final-RMSNormed in
// place by modules::lm_head, modules.hpp:242-246)
int ref_hidden_read(void *sp, float *out) {
	RefState *s = static_cast<RefState *>(sp);
	std::memcpy(out, s->d.xact.data.get(), sizeof(float) * s->m->cfg.hidden_size);
	return 0;
}

// ops.hpp:744
int ref_argmax_logits(const float *logits, int n) {
	(void)n;
	tensor::activation o(1, 1, constants::vocab);
	std::memcpy(o.data.get(), logits, sizeof(float) * constants::vocab);
	tensor::tokens t(1, 1);
	ops::argmax_logits(&t, &o);
	return t.data[0];
}

// ops.hpp:762; logits mutated in place into the reference's "probabilities"
int ref_minp_logits(float *logits, int n, float minp, float temp, float randf) {
	(void)n;
	tensor::activation o(1, 1, constants::vocab);
	std::memcpy(o.data.get(), logits, sizeof(float) * constants::vocab);
	tensor::tokens t(1, 1);
	ops::minp_logits(&t, &o, minp, temp, randf);
	std::memcpy(logits, o.data.get(), sizeof(float) * constants::vocab);
	return t.data[0];
}

// ops.hpp:634 linear_decode (y zeroed first, as modules.hpp does)
int ref_linear_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	return run_big_stack([&] {
		tensor::QuantArray q = borrow_weight(w, scales, K, N);
		tensor::activation a(1, 1, K), o(1, 1, N);
		std::memcpy(a.data.get(), x, sizeof(float) * K);
		ops::linear_decode(&o, &a, &q);
		std::memcpy(y, o.data.get(), sizeof(float) * N);
	});
}

// ops.hpp:654 lm_head_decode (row tile 4)
int ref_lm_head_decode(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	return run_big_stack([&] {
		tensor::QuantArray q = borrow_weight(w, scales, K, N);
		tensor::activation a(1, 1, K), o(1, 1, N);
		std::memcpy(a.data.get(), x, sizeof(float) * K);
		ops::lm_head_decode(&o, &a, &q);
		std::memcpy(y, o.data.get(), sizeof(float) * N);
	});
}

// ops.hpp:618 linear_prefill
int ref_linear_prefill(float *c, const float *a_in, const int8_t *w, const float *scales, int M, int K, int N) {
	return run_big_stack([&] {
		tensor::QuantArray q = borrow_weight(w, scales, K, N);
		// rows padded to a multiple of 32 floats is not needed: K,N are multiples of 32
		tensor::activation a(1, M, K), o(1, M, N);
		std::memcpy(a.data.get(), a_in, sizeof(float) * size_t(M) * K);
		ops::linear_prefill(&o, &a, &q);
		std::memcpy(c, o.data.get(), sizeof(float) * size_t(M) * N);
	});
}

// Timed loop for the isolated-op CPU baseline: `reps` calls of linear_decode
// (M==1, N!=vocab), lm_head_decode (M==1, N==vocab) or linear_prefill (M>1)
// on the same buffers; returns seconds via *secs.
int ref_time_linear(const float *x, const int8_t *w, const float *scales, int M, int K, int N, int reps, double *secs) {
	return run_big_stack([&] {
		tensor::QuantArray q = borrow_weight(w, scales, K, N);
		tensor::activation a(1, M, K), o(1, M, N);
		std::memcpy(a.data.get(), x, sizeof(float) * size_t(M) * K);
		auto t0 = std::chrono::high_resolution_clock::now();
		for (int r = 0; r < reps; r++) {
			if (M == 1) {
				o.zero();
				if (N == int(constants::vocab))
					ops::lm_head_decode(&o, &a, &q);
				else
					ops::linear_decode(&o, &a, &q);
			} else {
				ops::linear_prefill(&o, &a, &q);
			}
		}
		auto t1 = std::chrono::high_resolution_clock::now();
		*secs = (t1 - t0).count() / 1e9;
	});
}

// ops.hpp:182 rmsnorm over `rows` rows of length dim (3-D activation [1,rows,dim])
int ref_rmsnorm(float *x, const float *w, int rows, int dim) {
	return run_big_stack([&] {
		tensor::activation a(1, rows, dim);
		std::memcpy(a.data.get(), x, sizeof(float) * size_t(rows) * dim);
		tensor::FloatArray fw = make_f(w, dim);
		ops::rmsnorm(&a, &fw);
		std::memcpy(x, a.data.get(), sizeof(float) * size_t(rows) * dim);
	});
}

// decode.hpp:118 RoPE tables, [max_pos, head_dim] each
int ref_rope_tables(const char *size, int is_local, float *cos_out, float *sin_out) {
	return run_big_stack([&] {
		config::Config cfg = config::CONFIG_MAP.at(size);
		decode::RoPE r(&cfg, is_local != 0);
		size_t n = size_t(cfg.n_pos) * cfg.head_dim;
		std::memcpy(cos_out, r.freqs_cos.data.get(), sizeof(float) * n);
		std::memcpy(sin_out, r.freqs_sin.data.get(), sizeof(float) * n);
	});
}

// ops.hpp:29 GeLUTable
int ref_gelu_table(float mn, float mx, int size, float *out) {
	lut::GeLUTable t(mn, mx, size);
	std::memcpy(out, t.table.get(), sizeof(float) * size);
	return 0;
}

// The state's own tables, for upload into the product (so both sides use
// bit-identical cos/sin/GeLU tables and the comparison isolates the kernels).
int ref_state_tables(void *sp, float *cos_g, float *sin_g, float *cos_l, float *sin_l, float *gelu) {
	RefState *s = static_cast<RefState *>(sp);
	size_t n = size_t(s->m->cfg.n_pos) * s->m->cfg.head_dim;
	if (cos_g) std::memcpy(cos_g, s->rope.freqs_cos.data.get(), sizeof(float) * n);
	if (sin_g) std::memcpy(sin_g, s->rope.freqs_sin.data.get(), sizeof(float) * n);
	if (cos_l) std::memcpy(cos_l, s->rope_sw.freqs_cos.data.get(), sizeof(float) * n);
	if (sin_l) std::memcpy(sin_l, s->rope_sw.freqs_sin.data.get(), sizeof(float) * n);
	if (gelu) std::memcpy(gelu, s->table.table.get(), sizeof(float) * s->table.table_size);
	return 0;
}

// modules.hpp:203 mlp on x[S, D] in place. Weights in reference order:
// Up [D,I]+s, Gate [D,I]+s, Down [I,D]+s, pre-norm [D], post-norm [D].
int ref_module_mlp(float *x, int S, int D, int I, const int8_t *uw, const float *us, const int8_t *gw, const float *gs,
                   const int8_t *dw, const float *ds, const float *pre, const float *post, int gelu_size) {
	return run_big_stack([&] {
		config::Config cfg = config::CONFIG_MAP.at(D == 640 ? "270m" : "1B");
		modules::MLPLayer l(D, I);
		l.Uw = borrow_weight(uw, us, D, I);
		l.Gw = borrow_weight(gw, gs, D, I);
		l.Dw = borrow_weight(dw, ds, I, D);
		l.RMSw_pre = make_f(pre, D);
		l.RMSw_post = make_f(post, D);
		lut::GeLUTable table(-4.0, 4.0, gelu_size);
		tensor::activation a(1, S, D);
		std::memcpy(a.data.get(), x, sizeof(float) * size_t(S) * D);
		if (S > 1) {
			decode::PrefillState pf(1, S, &cfg);
			modules::mlp(&a, &l, nullptr, &pf, &table);
		} else {
			decode::DecodeState d(1, &cfg);
			modules::mlp(&a, &l, &d, nullptr, &table);
		}
		std::memcpy(x, a.data.get(), sizeof(float) * size_t(S) * D);
	});
}

// modules.hpp:89 attention on x[S, D] in place. If n_cached > 0, S must be 1 and
// the cache is pre-filled with k_cache/v_cache [n_cached, 256] (already
// normed+roped keys), position_ptr = buffer_ptr = n_cached — the set-up of the
// reference's attention_decode unit test (tests/csrc/test_bench_modules.cpp:108).
int ref_module_attention(float *x, int S, int D, int is_sw, const int8_t *qw, const float *qs, const int8_t *kw,
                         const float *ks, const int8_t *vw, const float *vs, const int8_t *ow, const float *os,
                         const float *rmsq, const float *rmsk, const float *pre, const float *post, int n_cached,
                         const float *k_cache, const float *v_cache) {
	return run_big_stack([&] {
		config::Config cfg = config::CONFIG_MAP.at(D == 640 ? "270m" : "1B");
		int qd = cfg.n_head * cfg.head_dim, kd = cfg.n_kv * cfg.head_dim;
		modules::AttentionLayer l(D, cfg.head_dim, cfg.n_head, cfg.n_kv, is_sw != 0);
		l.Qw = borrow_weight(qw, qs, D, qd);
		l.Kw = borrow_weight(kw, ks, D, kd);
		l.Vw = borrow_weight(vw, vs, D, kd);
		l.Ow = borrow_weight(ow, os, qd, D);
		l.RMSq = make_f(rmsq, cfg.head_dim);
		l.RMSk = make_f(rmsk, cfg.head_dim);
		l.RMSw_pre = make_f(pre, D);
		l.RMSw_post = make_f(post, D);
		decode::KVCache kv(1, &cfg, is_sw != 0);
		decode::RoPE rope(&cfg, is_sw != 0);
		tensor::activation a(1, S, D);
		std::memcpy(a.data.get(), x, sizeof(float) * size_t(S) * D);
		if (S > 1) {
			decode::PrefillState pf(1, S, &cfg);
			modules::attention(&a, &l, nullptr, &kv, &pf, &rope);
		} else {
			if (n_cached > 0) {
				std::memcpy(kv.keys.data.get(), k_cache, sizeof(float) * size_t(n_cached) * cfg.head_dim);
				std::memcpy(kv.values.data.get(), v_cache, sizeof(float) * size_t(n_cached) * cfg.head_dim);
				kv.position_ptr = n_cached;
				kv.buffer_ptr = n_cached;
			}
			decode::DecodeState d(1, &cfg);
			modules::attention(&a, &l, &d, &kv, nullptr, &rope);
		}
		std::memcpy(x, a.data.get(), sizeof(float) * size_t(S) * D);
	});
}

// modules.hpp:223 lm_head on x[S, D] -> logits[V]
int ref_module_lm_head(float *logits, const float *x, int S, int D, const int8_t *w, const float *scales,
                       const float *rmsw) {
	return run_big_stack([&] {
		tensor::QuantArray q = borrow_weight(w, scales, D, constants::vocab);
		tensor::FloatArray fw = make_f(rmsw, D);
		tensor::activation a(1, S, D), o(1, 1, constants::vocab);
		std::memcpy(a.data.get(), x, sizeof(float) * size_t(S) * D);
		modules::lm_head(&o, &a, &q, &fw);
		std::memcpy(logits, o.data.get(), sizeof(float) * constants::vocab);
	});
}

}  // extern "C"
