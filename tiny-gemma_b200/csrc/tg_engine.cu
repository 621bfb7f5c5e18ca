// libtinygemma_b200: host-side engine and the extern "C" boundary declared in
// include/tiny_gemma_b200.h. Owns the device weight store (gemma_i8.bin bytes
// unchanged in HBM), the per-state KV caches and scratch, the launch plans and
// the CUDA graph of one decode step.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <string>
#include <vector>

#include "../../include/tiny_gemma_b200.h"
#include "kernels_decode.cuh"
#include "kernels_mega.cuh"
#include "kernels_persist.cuh"
#include "kernels_gemm_tc.cuh"
#include "kernels_attn_tc.cuh"
#include "kernels_prefill.cuh"
#include "kernels_sampler.cuh"

using namespace tg;

// ===================================================================== errors
namespace {

thread_local std::string g_err;
std::atomic<long long> g_launches{0};

int fail(int code, const std::string &msg) {
	g_err = msg;
	return code;
}

#define TG_CUDA(call)                                                                                   \
	do {                                                                                                \
		cudaError_t e__ = (call);                                                                       \
		if (e__ != cudaSuccess)                                                                         \
			return fail(TG_ECUDA, std::string(#call) + ": " + cudaGetErrorString(e__));                 \
	} while (0)

#define TG_TRY(call)                \
	do {                            \
		int rc__ = (call);          \
		if (rc__ != TG_OK) return rc__; \
	} while (0)

inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char *what) {
	cudaError_t e = cudaGetLastError();
	if (e != cudaSuccess) return fail(TG_ECUDA, std::string(what) + " launch: " + cudaGetErrorString(e));
	return TG_OK;
}

// tunables (set through the environment for experiments; defaults are the tuned values)
int env_int(const char *name, int dflt) {
	const char *v = std::getenv(name);
	return v ? std::atoi(v) : dflt;
}

int g_num_sms = 148;

// cudaFuncSetAttribute is per device: "configured once" flags are kept per device index
constexpr int TG_MAX_DEVICES = 64;
// Launch with the programmatic-serialization attribute (see pdl_wait in tg_common.cuh): only for kernels that
// call pdl_wait() before their first global access. TG_PDL=0 launches them as ordinary stream-ordered kernels.
// The batched decode step switches it off for its own launches (g_pdl_scope_off): replayed from a CUDA graph the
// step gains nothing from it (measured 3.72 ms with ordinary edges, 3.78 ms with programmatic ones at 256
// sequences), while the eagerly launched prefill does (178 tokens: 4.00 -> 3.80 ms).
thread_local bool g_pdl_scope_off = false;
template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
	static const int use_env = env_int("TG_PDL", 1);
	const int use = use_env && !g_pdl_scope_off;
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid;
	cfg.blockDim = block;
	cfg.dynamicSmemBytes = smem;
	cfg.stream = st;
	cudaLaunchAttribute at[1];
	at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	at[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = at;
	cfg.numAttrs = use ? 1 : 0;
	cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // errors surface in check_launch (cudaGetLastError)
}

inline int current_device_slot() {
	int d = 0;
	cudaGetDevice(&d);
	return (d >= 0 && d < TG_MAX_DEVICES) ? d : 0;
}

}  // namespace

// ===================================================================== model
struct QW {
	const int8_t *q = nullptr;
	const float *s = nullptr;
	int K = 0, N = 0;
	int ld = 0;  // bytes between rows when the matrix is a column slice of a wider one; 0: N
};

struct LayerW {
	QW Q, K, V, O, U, G, Dn;
	const float *rmsq, *rmsk, *attn_pre, *attn_post, *mlp_pre, *mlp_post;
	bool is_local;
};

struct tg_model {
	tg_config cfg;
	int device = 0;
	long weights_version = 0;  // bumped by every load
	// layer weights re-ordered into the persistent decode kernel's per-CTA units (built on first use)
	int8_t *dec_tiled = nullptr;
	size_t dec_tiled_bytes = 0;
	long dec_tiled_version = -1;
	int dec_tiled_key[12] = {0};
	// the same for the dp4a decode kernel: layer units as 4 x 4 pieces, and the lm_head in ring-stage order
	int8_t *ps_tiled = nullptr, *ps_lm = nullptr;
	size_t ps_tiled_bytes = 0, ps_lm_bytes = 0;
	long ps_tiled_version = -1;
	int ps_tiled_key[20] = {0};
	uint8_t *blob = nullptr;
	size_t nbytes = 0;
	const int8_t *wte = nullptr;
	const float *wte_s = nullptr, *final_norm = nullptr;
	std::vector<LayerW> layers;
	QW lm_head;
	float *rope[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}};  // [is_local][cos,sin]
	int rope_npos[2] = {0, 0};
	float *gelu = nullptr;
	float gelu_min = -4.0f, gelu_max = 4.0f, gelu_eps = 0.0f;
	int gelu_size = 0;
	bool loaded = false;
};

namespace {

size_t model_file_bytes(const tg_config &c) {
	size_t qd = size_t(c.n_head) * c.head_dim, kd = size_t(c.n_kv) * c.head_dim;
	size_t D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	size_t per_layer = (D * qd + 4 * qd) + 2 * (D * kd + 4 * kd) + (qd * D + 4 * D) + 2 * 4 * size_t(c.head_dim) +
	                   2 * 4 * D + 2 * (D * I + 4 * I) + (I * D + 4 * D) + 2 * 4 * D;
	return V * D + 4 * D + 4 * D + size_t(c.n_layers) * per_layer + D * V + 4 * V;
}

// transformer.hpp:99-165 read order; pointers into the device blob
void bind_model(tg_model *m) {
	const tg_config &c = m->cfg;
	const uint8_t *p = m->blob;
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
	const int D = c.hidden_size, I = c.intermediate_size, qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	m->wte = reinterpret_cast<const int8_t *>(take(size_t(c.n_vocab) * D));
	m->wte_s = takef(D);
	m->final_norm = takef(D);
	m->layers.resize(c.n_layers);
	for (int l = 0; l < c.n_layers; l++) {
		LayerW &w = m->layers[l];
		w.Q = takeq(D, qd);
		w.K = takeq(D, kd);
		w.V = takeq(D, kd);
		w.O = takeq(qd, D);
		w.rmsq = takef(c.head_dim);
		w.rmsk = takef(c.head_dim);
		w.attn_pre = takef(D);
		w.attn_post = takef(D);
		w.U = takeq(D, I);
		w.G = takeq(D, I);
		w.Dn = takeq(I, D);
		w.mlp_pre = takef(D);
		w.mlp_post = takef(D);
		w.is_local = (l % c.window_pattern) != (c.window_pattern - 1);  // transformer.hpp:43
	}
	m->lm_head = takeq(D, c.n_vocab);
}

bool supported_k(int K) { return K == 640 || K == 2048 || K == 1024 || K == 256 || K == 1152 || K == 6912; }
bool supported_n(int N) {
	return N == 640 || N == 262144 || N == 2048 || N == 256 || N == 1024 || N == 1152 || N == 6912;
}

int ensure_device(int device) {
	int n = 0;
	cudaError_t e = cudaGetDeviceCount(&n);
	if (e != cudaSuccess || n == 0) {
		cudaGetLastError();
		return fail(TG_ENODEVICE, "no CUDA device available (this library has no CPU path)");
	}
	if (device < 0 || device >= n) return fail(TG_EINVAL, "device index out of range");
	TG_CUDA(cudaSetDevice(device));
	int sms = 0;
	if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && sms > 0) g_num_sms = sms;
	return TG_OK;
}

// ------------------------------------------------------------- matvec planning
struct MvPlan {
	int nsplit, kc, grid_x;
};

// Pick the K-split so that the launch fills the GPU in whole waves. kc must be a
// multiple of 32 rows and divide K.
MvPlan plan_matvec(int K, int ntiles, int target_ctas, int max_split = 1 << 30) {
	MvPlan best{1, K, ntiles};
	if (ntiles >= target_ctas) return best;
	double best_score = -1e9;
	const int units = K / 32;
	for (int ns = 1; ns <= units && ns <= max_split; ns++) {
		if (units % ns) continue;
		int ctas = ntiles * ns;
		int waves = (ctas + g_num_sms - 1) / g_num_sms;
		double eff = double(ctas) / (double(waves) * g_num_sms);
		double fill = std::min(1.0, double(ctas) / target_ctas);
		double score = eff * fill - 0.01 * std::log2(double(ns));
		if (score > best_score) {
			best_score = score;
			best = MvPlan{ns, K / ns, ntiles};
		}
	}
	return best;
}

size_t mv_smem_bytes(int MB, int pro, int epi, int K, int kc) {
	size_t f = size_t(MB) * kc;
	if (pro != PRO_PLAIN) f += size_t(MB) * K;
	f += size_t(MB) * MV_NWARPS * MV_TN * (epi == EPI_GEGLU ? 2 : 1);
	return f * sizeof(float);
}

template <int MB, int PRO, int EPI>
int launch_mv_t(const MvArgs &a, dim3 grid, size_t smem, cudaStream_t st) {
	static size_t configured[TG_MAX_DEVICES] = {0};
	const int dev = current_device_slot();
	if (smem > 48 * 1024 && smem > configured[dev]) {
		TG_CUDA(cudaFuncSetAttribute(qmatvec_kernel<MB, PRO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
		configured[dev] = smem;
	}
	qmatvec_kernel<MB, PRO, EPI><<<grid, MV_THREADS, smem, st>>>(a);
	count_launch();
	return check_launch("qmatvec");
}

template <int MB>
int launch_mv_b(const MvArgs &a, int pro, int epi, dim3 grid, size_t smem, cudaStream_t st) {
	if (epi == EPI_GEGLU) {
		if (pro == PRO_RESNORM) return launch_mv_t<MB, PRO_RESNORM, EPI_GEGLU>(a, grid, smem, st);
		if (pro == PRO_NORM) return launch_mv_t<MB, PRO_NORM, EPI_GEGLU>(a, grid, smem, st);
		return launch_mv_t<MB, PRO_PLAIN, EPI_GEGLU>(a, grid, smem, st);
	}
	if (pro == PRO_RESNORM) return launch_mv_t<MB, PRO_RESNORM, EPI_SCALE>(a, grid, smem, st);
	if (pro == PRO_NORM) return launch_mv_t<MB, PRO_NORM, EPI_SCALE>(a, grid, smem, st);
	return launch_mv_t<MB, PRO_PLAIN, EPI_SCALE>(a, grid, smem, st);
}

// a.B may be 1..4 per launch
int launch_mv(MvArgs a, int pro, int epi, cudaStream_t st) {
	dim3 grid(std::min(a.ntiles, 65535), a.nsplit);
	const int MB = a.B <= 1 ? 1 : (a.B == 2 ? 2 : 4);
	size_t smem = mv_smem_bytes(MB, pro, epi, a.K, a.kc);
	switch (MB) {
		case 1:
			return launch_mv_b<1>(a, pro, epi, grid, smem, st);
		case 2:
			return launch_mv_b<2>(a, pro, epi, grid, smem, st);
		default:
			return launch_mv_b<4>(a, pro, epi, grid, smem, st);
	}
}

constexpr int MV_MAX_B = 4;
constexpr int STEP_RANDF = 64;  // uniforms per sequence that fit the state's step block (more: a buffer of their own)

// Single-wave matvec (qmatvec_cluster_kernel): a [K, N] matrix qualifies when a tile width 16 * tpr and a
// K-split ks (= cluster size) exist with all CTAs resident at once — one per SM, and no more clusters than
// the device can hold at a time (a cluster needs its SMs inside one GPC) — and at most MVC_MAX_IT rows per
// thread. Among those the plan with the most CTAs wins, then the smaller cluster, then the wider tile.
struct MvcPlan {
	int tpr = 0, ks = 0, nt = 512;
};
template <int TPR, int NT>
int mvc_launch_t(float *y, const float *x, const int8_t *w, const float *scales, int K, int N, int ks, cudaStream_t st, int *max_clusters) {
	cudaLaunchConfig_t cfg{};
	cfg.gridDim = dim3(N / (16 * TPR), ks);
	cfg.blockDim = dim3(NT);
	cfg.dynamicSmemBytes = 0;
	cfg.stream = st;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = 1;
	attr[0].val.clusterDim.y = unsigned(ks);
	attr[0].val.clusterDim.z = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	if (max_clusters) {  // query only
		TG_CUDA(cudaOccupancyMaxActiveClusters(max_clusters, qmatvec_cluster_kernel<TPR, NT>, &cfg));
		return TG_OK;
	}
	TG_CUDA(cudaLaunchKernelEx(&cfg, qmatvec_cluster_kernel<TPR, NT>, y, x, w, scales, K, N, K / ks));
	count_launch();
	return check_launch("qmatvec_cluster");
}
int mvc_launch(MvcPlan p, float *y, const float *x, const int8_t *w, const float *scales, int K, int N, cudaStream_t st, int *max_clusters = nullptr) {
	if (p.nt == 256) {
		if (p.tpr == 1) return mvc_launch_t<1, 256>(y, x, w, scales, K, N, p.ks, st, max_clusters);
		if (p.tpr == 2) return mvc_launch_t<2, 256>(y, x, w, scales, K, N, p.ks, st, max_clusters);
		return mvc_launch_t<4, 256>(y, x, w, scales, K, N, p.ks, st, max_clusters);
	}
	if (p.tpr == 1) return mvc_launch_t<1, 512>(y, x, w, scales, K, N, p.ks, st, max_clusters);
	if (p.tpr == 2) return mvc_launch_t<2, 512>(y, x, w, scales, K, N, p.ks, st, max_clusters);
	return mvc_launch_t<4, 512>(y, x, w, scales, K, N, p.ks, st, max_clusters);
}
MvcPlan mvc_plan(int K, int N, int dev) {
	// clusters of each (tile width, size) the device holds at once: asked once per device
	static int max_active[TG_MAX_DEVICES][2][3][4];  // [256 / 512 threads][tile width][cluster size]
	static bool asked[TG_MAX_DEVICES] = {false};
	const int slot = (dev >= 0 && dev < TG_MAX_DEVICES) ? dev : 0;
	if (!asked[slot]) {
		for (int h = 0; h < 2; h++)
			for (int t = 0; t < 3; t++)
				for (int c = 0; c < 4; c++) {
					int n = 0;
					// (grid of one cluster: the answer does not depend on the grid)
					if (mvc_launch(MvcPlan{1 << t, 1 << c, h ? 512 : 256}, nullptr, nullptr, nullptr, nullptr, 1 << c, 16 << t, nullptr, &n) != TG_OK) n = 0;
					max_active[slot][h][t][c] = n;
				}
		asked[slot] = true;
	}
	const int want_tpr = env_int("TG_MVC_TPR", 0), want_ks = env_int("TG_MVC_KS", 0), want_nt = env_int("TG_MVC_NT", 0);  // (experiments: fix the plan)
	// CTAs of 256 threads where a plan exists with them (the small matrices: 3.5 - 4.2 us against 4.1 - 5.0 with 512:
	// half the warps to launch and to reduce over); 512 threads reach K-slices of up to 1280 rows per 16 columns
	MvcPlan best;
	for (int nt : {256, 512}) {
		if (want_nt && nt != want_nt) continue;
		int best_ctas = 0;
		for (int c = 0; c < 4; c++)          // smaller clusters first
			for (int t = 2; t >= 0; t--) {   // wider tiles first
				const int tpr = 1 << t, ks = 1 << c, tn = 16 * tpr;
				if (want_tpr && tpr != want_tpr) continue;
				if (want_ks && ks != want_ks) continue;
				if (N % tn != 0 || K % ks != 0) continue;
				const int tiles = N / tn, kc = K / ks;
				if (kc > MVC_MAX_IT * (nt / tpr)) continue;
				// (one CTA per SM: 256-thread CTAs fit three to an SM, but two resident waves of them measured slower on
				// five of the six layer shapes; TG_MVC_WAVES=2 allows them)
				if (tiles * ks > (nt == 256 ? env_int("TG_MVC_WAVES", 1) : 1) * g_num_sms || tiles > max_active[slot][nt == 512][t][c]) continue;
				if (tiles * ks > best_ctas) {
					best_ctas = tiles * ks;
					best = MvcPlan{tpr, ks, nt};
				}
			}
		if (best.ks) break;
	}
	return best;
}

}  // namespace

// ------------------------------------------------------------- prefill
// Tensor-core GEMM (kernels_gemm_tc.cuh): activations are split into three bf16 terms and packed
// tile by tile once per distinct A (pack_activations), then any number of weight matrices with
// the same K can be multiplied against that packing (launch_gemm_tc).
struct TcScratch {
	__nv_bfloat16 *apack = nullptr;
	size_t apack_bytes = 0;
	float *partial = nullptr;  // split-K partial sums
	size_t partial_floats = 0;
	unsigned *tickets = nullptr;  // [TC_TICKETS] zeros: enables the in-kernel split-K reduction for shallow splits
	int fused_max_split = 3;      // deeper splits use the reduce kernel: one CTA re-reading a whole tile of every split is
	                              // latency-bound (measured: 9-way splits reduced in-kernel doubled the batched step time)
	int max_split = 9;            // cap on the K-split depth: deeper splits (one or two K-blocks per CTA) cost more in partial-sum
	                              // traffic and per-CTA fixed cost than they gain in parallelism (TG_GEMM_MAX_SPLIT overrides)
	unsigned long long *top1 = nullptr;  // set for one launch: row-wise (max, column) keys instead of C (unsplit K)
	int top1_col0 = 0;
	int *err = nullptr;
};

// ===================================================================== state
struct tg_state {
	tg_model *m = nullptr;
	int B = 1;
	int max_pos_global = 0;
	cudaStream_t stream = nullptr;
	// per-layer caches
	std::vector<float *> kcache, vcache;  // [B][slots][256]
	std::vector<int> slots;
	// decode activations
	float *h[2] = {nullptr, nullptr};  // residual stream ping-pong [B][D]
	float *qkv = nullptr;              // [B][qd+2kd]
	float *attn_out = nullptr;         // [B][qd]
	float *t = nullptr;                // [B][D]
	float *act = nullptr;              // [B][I]
	float *xnorm = nullptr;            // [B][D] final-normed hidden (parity read-back)
	float *logits = nullptr;           // [B][V]
	float *partial = nullptr;          // split-K scratch
	size_t partial_floats = 0;
	unsigned *tickets = nullptr;       // [max tiles] + [B] for attention
	unsigned *attn_tickets = nullptr;
	float *attn_part = nullptr;        // [B][nsplit_max][1032]
	int attn_nsplit_local = 16, attn_nsplit_global = 64;
	int *step_pos = nullptr, *next_pos = nullptr, *ring_base = nullptr;  // [B]
	int *tok = nullptr;                // [B]
	int *tok_log = nullptr;            // [log_cap][B]
	int *force_ids = nullptr;          // [force_cap] tokens of tg_append (batch 1)
	int force_cap = 0;
	int log_cap = 0;
	int *log_count = nullptr;          // [B]
	float *randf = nullptr;            // [randf_cap][B]
	int randf_cap = 0;
	int randf_valid = 0;               // uniforms per sequence uploaded so far (the largest upload)
	// One allocation holds the small per-step words, so that a step's inputs go up in ONE copy and its
	// results come back in ONE: [err_flag, 3 pad][tok B][randf_count B][log_count B][randf STEP_RANDF x B]
	int *step_blk = nullptr;
	bool randf_in_blk = false;         // randf still points into step_blk (it moves out when it has to grow)
	float *randf_blk = nullptr;        // the block's own STEP_RANDF x B uniforms
	bool lean_randf = false;           // the next persistent launch draws from randf_blk (one-token calls)
	// persistent kernel: its hand-off arena and grid-barrier counter are left ready by the previous launch
	bool ps_clean = false;             // false: wipe the arena and zero the counter before the next launch
	unsigned ps_bar_base = 0;          // arrivals at the grid barrier so far
	int *randf_count = nullptr;        // [B]
	int *err_flag = nullptr;
	int *host_pin = nullptr;           // pinned staging, 64 KiB
	bool staging_busy = false;         // an enqueued copy may still read host_pin (set by the asynchronous tg_decode)
	// prefill scratch (grow-only)
	float *pf = nullptr;
	size_t pf_floats = 0;
	int *pf_ids = nullptr;
	int pf_ids_cap = 0;
	// plans
	MvPlan plan_qkv, plan_o, plan_gu, plan_dn, plan_lm;
	// decode graph
	cudaGraphExec_t graph = nullptr;
	bool use_graph = true;
	bool warmed = false;
	int graph_launches = 0;
	std::vector<int> host_pos;  // mirror of next_pos for call-order checks
	// batched decode step (tensor-core GEMMs with M = batch)
	bool batched_ok = false;
	float *bx = nullptr, *bup = nullptr;  // [B][D] normed input, [B][I] up projection
	TcScratch btc;
	// persistent decode kernel (batch 1)
	bool mega_ok = false;
	MgArgs mega{};
	CUtensorMap *d_tmaps = nullptr;
	MgLayer *d_layers = nullptr;
	float *mg_ll = nullptr, *mg_samp_f = nullptr, *mg_probs = nullptr;
	uint2 *mg_pe = nullptr;
	unsigned mg_seq = 0;  // layer tags consumed so far by the tagged hand-off
	size_t mg_ll_bytes = 0;
	int *mg_samp_i = nullptr;
	unsigned *mg_bar = nullptr;
	int mega_grid = 0;
	long long *mg_dbg = nullptr;
	// dp4a persistent decode kernel
	bool ps_ok = false;
	PsArgs ps{};
	PsLayer *d_pslayers = nullptr;
	float *ps_ll = nullptr;
	size_t ps_ll_bytes = 0;
	size_t mega_smem = 0;
};

namespace {

int state_alloc(tg_state *s) {
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int B = s->B, D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	TG_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
	s->kcache.resize(c.n_layers);
	s->vcache.resize(c.n_layers);
	s->slots.resize(c.n_layers);
	for (int l = 0; l < c.n_layers; l++) {
		int slots = m->layers[l].is_local ? c.n_pos_local : s->max_pos_global;
		s->slots[l] = slots;
		size_t n = size_t(B) * slots * c.head_dim * c.n_kv;
		TG_CUDA(cudaMalloc(&s->kcache[l], n * 4));
		TG_CUDA(cudaMalloc(&s->vcache[l], n * 4));
		TG_CUDA(cudaMemsetAsync(s->kcache[l], 0, n * 4, s->stream));
		TG_CUDA(cudaMemsetAsync(s->vcache[l], 0, n * 4, s->stream));
	}
	auto allocf = [&](float **p, size_t n) -> int {
		TG_CUDA(cudaMalloc(p, n * 4));
		TG_CUDA(cudaMemsetAsync(*p, 0, n * 4, s->stream));
		return TG_OK;
	};
	TG_TRY(allocf(&s->h[0], size_t(B) * D));
	TG_TRY(allocf(&s->h[1], size_t(B) * D));
	TG_TRY(allocf(&s->qkv, size_t(B) * (qd + 2 * kd)));
	TG_TRY(allocf(&s->attn_out, size_t(B) * qd));
	TG_TRY(allocf(&s->t, size_t(B) * D));
	TG_TRY(allocf(&s->act, size_t(B) * I));
	TG_TRY(allocf(&s->xnorm, size_t(B) * D));
	TG_TRY(allocf(&s->logits, size_t(B) * V));

	const int target = env_int("TG_MV_TARGET_CTAS", 2 * g_num_sms);
	s->plan_qkv = plan_matvec(D, (qd + 2 * kd) / MV_TN, target);
	s->plan_o = plan_matvec(qd, D / MV_TN, target);
	s->plan_gu = plan_matvec(D, I / MV_TN, target);
	s->plan_dn = plan_matvec(I, D / MV_TN, target);
	s->plan_lm = plan_matvec(D, V / MV_TN, target);
	const int mb = std::min(B, MV_MAX_B);
	size_t pf = 0;
	pf = std::max(pf, size_t(s->plan_qkv.nsplit) * mb * (qd + 2 * kd));
	pf = std::max(pf, size_t(s->plan_o.nsplit) * mb * D);
	pf = std::max(pf, size_t(s->plan_gu.nsplit) * mb * 2 * I);
	pf = std::max(pf, size_t(s->plan_dn.nsplit) * mb * D);
	s->partial_floats = pf;
	TG_TRY(allocf(&s->partial, pf));
	TG_CUDA(cudaMalloc(&s->tickets, sizeof(unsigned) * (V / MV_TN)));
	TG_CUDA(cudaMemsetAsync(s->tickets, 0, sizeof(unsigned) * (V / MV_TN), s->stream));
	TG_CUDA(cudaMalloc(&s->attn_tickets, sizeof(unsigned) * B));
	TG_CUDA(cudaMemsetAsync(s->attn_tickets, 0, sizeof(unsigned) * B, s->stream));
	// split-KV factor: enough CTAs (batch x splits) to fill the GPU about three times, no more —
	// every split repeats the q/k norm + RoPE and adds a partial to merge
	auto pick_split = [&](int cap) {
		int ns = 1;
		while (ns < cap && B * ns < 3 * g_num_sms) ns *= 2;
		return ns;
	};
	s->attn_nsplit_local = env_int("TG_ATTN_SPLIT_LOCAL", pick_split(16));
	s->attn_nsplit_global = env_int("TG_ATTN_SPLIT_GLOBAL", pick_split(64));
	int nsmax = std::max(s->attn_nsplit_local, s->attn_nsplit_global);
	TG_TRY(allocf(&s->attn_part, size_t(B) * nsmax * (AT_NH * AT_HD + 8)));
	auto alloci = [&](int **p, size_t n) -> int {
		TG_CUDA(cudaMalloc(p, n * 4));
		TG_CUDA(cudaMemsetAsync(*p, 0, n * 4, s->stream));
		return TG_OK;
	};
	TG_TRY(alloci(&s->step_pos, B));
	TG_TRY(alloci(&s->next_pos, B));
	TG_TRY(alloci(&s->ring_base, B));
	TG_TRY(alloci(&s->step_blk, 4 + size_t(3 + STEP_RANDF) * B));
	s->err_flag = s->step_blk;
	s->tok = s->step_blk + 4;
	s->randf_count = s->tok + B;
	s->log_count = s->randf_count + B;
	s->randf_blk = reinterpret_cast<float *>(s->log_count + B);
	s->randf = s->randf_blk;
	s->randf_cap = STEP_RANDF;
	s->randf_in_blk = true;
	TG_CUDA(cudaMallocHost(&s->host_pin, 64 * 1024));
	s->host_pos.assign(B, 0);
	s->use_graph = env_int("TG_USE_GRAPH", 1) != 0;
	TG_CUDA(cudaStreamSynchronize(s->stream));
	return TG_OK;
}

GeluLut make_lut(const tg_model *m) { return GeluLut{m->gelu, m->gelu_min, m->gelu_eps, m->gelu_size}; }

int check_ready(const tg_model *m) {
	if (!m->rope[0][0] || !m->rope[1][0] || !m->gelu)
		return fail(TG_ESTATE, "RoPE / GeLU tables not set (tg_model_set_rope, tg_model_set_gelu_table or tg_model_build_tables)");
	return TG_OK;
}

// ------------------------------------------------------------- decode step
// One token for sequences [b0, b0+nb) (nb <= MV_MAX_B). Kernel sequence per
// layer: QKV matvec (norm prologue) -> attention -> O matvec -> gate/up matvec
// (residual+norm prologue, GeGLU epilogue) -> down matvec; then the lm_head
// matvec with the last residual+norm prologue.
int enqueue_decode_chunk(tg_state *s, int b0, int nb, bool with_lm_head = true) {
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	cudaStream_t st = s->stream;
	const GeluLut lut = make_lut(m);

	EmbedArgs ea;
	ea.wte = m->wte;
	ea.scales = m->wte_s;
	ea.tok = s->tok + b0;
	ea.h = s->h[0] + size_t(b0) * D;
	ea.step_pos = s->step_pos + b0;
	ea.next_pos = s->next_pos + b0;
	ea.err_flag = s->err_flag;
	ea.D = D;
	ea.V = V;
	ea.sqrtD = float(std::sqrt(double(D)));  // ops.hpp:584 `const float scale = sqrt(dims)`
	embed_decode_kernel<<<nb, 256, 0, st>>>(ea);
	count_launch();
	TG_TRY(check_launch("embed_decode"));

	int cur = 0;  // index of the buffer holding the residual stream
	for (int l = 0; l < c.n_layers; l++) {
		const LayerW &w = m->layers[l];
		// ---- QKV
		{
			MvArgs a{};
			a.seg[0] = MvSeg{w.Q.q, w.Q.s, qd, 0, 0};
			a.seg[1] = MvSeg{w.K.q, w.K.s, kd, qd, qd / MV_TN};
			a.seg[2] = MvSeg{w.V.q, w.V.s, kd, qd + kd, (qd + kd) / MV_TN};
			a.nseg = 3;
			a.ntiles = (qd + 2 * kd) / MV_TN;
			a.K = D;
			a.kc = s->plan_qkv.kc;
			a.nsplit = s->plan_qkv.nsplit;
			a.B = nb;
			a.part_stride = qd + 2 * kd;
			a.out_stride = qd + 2 * kd;
			a.h = s->h[cur] + size_t(b0) * D;
			a.w_pre = w.attn_pre;
			a.partial = s->partial;
			a.tickets = s->tickets;
			a.out = s->qkv + size_t(b0) * (qd + 2 * kd);
			int pro = PRO_NORM;
			if (l > 0) {
				pro = PRO_RESNORM;
				a.t = s->t + size_t(b0) * D;
				a.w_post = m->layers[l - 1].mlp_post;
				a.h_out = s->h[cur ^ 1] + size_t(b0) * D;
			}
			TG_TRY(launch_mv(a, pro, EPI_SCALE, st));
			if (l > 0) cur ^= 1;
		}
		// ---- attention over the cache
		{
			AttnArgs a{};
			a.qkv = s->qkv + size_t(b0) * (qd + 2 * kd);
			a.rmsq = w.rmsq;
			a.rmsk = w.rmsk;
			a.cosT = m->rope[w.is_local ? 1 : 0][0];
			a.sinT = m->rope[w.is_local ? 1 : 0][1];
			a.slots = s->slots[l];
			a.kcache = s->kcache[l] + size_t(b0) * a.slots * AT_HD;
			a.vcache = s->vcache[l] + size_t(b0) * a.slots * AT_HD;
			a.is_local = w.is_local ? 1 : 0;
			a.step_pos = s->step_pos + b0;
			a.ring_base = s->ring_base + b0;
			a.nsplit = w.is_local ? s->attn_nsplit_local : s->attn_nsplit_global;
			a.part = s->attn_part + size_t(b0) * a.nsplit * (AT_NH * AT_HD + 8);
			a.tickets = s->attn_tickets + b0;
			a.out = s->attn_out + size_t(b0) * qd;
			a.err_flag = s->err_flag;
			attn_decode_kernel<<<dim3(a.nsplit, nb), AT_THREADS, 0, st>>>(a);
			count_launch();
			TG_TRY(check_launch("attn_decode"));
		}
		// ---- O projection
		{
			MvArgs a{};
			a.seg[0] = MvSeg{w.O.q, w.O.s, D, 0, 0};
			a.nseg = 1;
			a.ntiles = D / MV_TN;
			a.K = qd;
			a.kc = s->plan_o.kc;
			a.nsplit = s->plan_o.nsplit;
			a.B = nb;
			a.part_stride = D;
			a.out_stride = D;
			a.x = s->attn_out + size_t(b0) * qd;
			a.partial = s->partial;
			a.tickets = s->tickets;
			a.out = s->t + size_t(b0) * D;
			TG_TRY(launch_mv(a, PRO_PLAIN, EPI_SCALE, st));
		}
		// ---- gate/up with GeGLU
		{
			MvArgs a{};
			a.seg[0] = MvSeg{w.U.q, w.U.s, I, 0, 0};
			a.seg[1] = MvSeg{w.G.q, w.G.s, I, I, 0};
			a.nseg = 2;
			a.ntiles = I / MV_TN;
			a.K = D;
			a.kc = s->plan_gu.kc;
			a.nsplit = s->plan_gu.nsplit;
			a.B = nb;
			a.part_stride = 2 * I;
			a.out_stride = I;
			a.h = s->h[cur] + size_t(b0) * D;
			a.t = s->t + size_t(b0) * D;
			a.w_post = w.attn_post;
			a.w_pre = w.mlp_pre;
			a.h_out = s->h[cur ^ 1] + size_t(b0) * D;
			a.partial = s->partial;
			a.tickets = s->tickets;
			a.out = s->act + size_t(b0) * I;
			a.lut = lut;
			TG_TRY(launch_mv(a, PRO_RESNORM, EPI_GEGLU, st));
			cur ^= 1;
		}
		// ---- down projection
		{
			MvArgs a{};
			a.seg[0] = MvSeg{w.Dn.q, w.Dn.s, D, 0, 0};
			a.nseg = 1;
			a.ntiles = D / MV_TN;
			a.K = I;
			a.kc = s->plan_dn.kc;
			a.nsplit = s->plan_dn.nsplit;
			a.B = nb;
			a.part_stride = D;
			a.out_stride = D;
			a.x = s->act + size_t(b0) * I;
			a.partial = s->partial;
			a.tickets = s->tickets;
			a.out = s->t + size_t(b0) * D;
			TG_TRY(launch_mv(a, PRO_PLAIN, EPI_SCALE, st));
		}
	}
	if (!with_lm_head) {
		final_hidden_kernel<<<nb, 256, size_t(D) * 4, st>>>(s->xnorm + size_t(b0) * D, s->h[cur] + size_t(b0) * D,
		                                                    s->t + size_t(b0) * D, m->layers[c.n_layers - 1].mlp_post,
		                                                    m->final_norm, D);
		count_launch();
		return check_launch("final_hidden");
	}
	// ---- lm_head (final residual add + final norm in the prologue)
	{
		MvArgs a{};
		a.seg[0] = MvSeg{m->lm_head.q, m->lm_head.s, V, 0, 0};
		a.nseg = 1;
		a.ntiles = V / MV_TN;
		a.K = D;
		a.kc = s->plan_lm.kc;
		a.nsplit = s->plan_lm.nsplit;
		a.B = nb;
		a.part_stride = V;
		a.out_stride = V;
		a.h = s->h[cur] + size_t(b0) * D;
		a.t = s->t + size_t(b0) * D;
		a.w_post = m->layers[c.n_layers - 1].mlp_post;
		a.w_pre = m->final_norm;
		a.h_out = s->h[cur ^ 1] + size_t(b0) * D;
		a.x_out = s->xnorm + size_t(b0) * D;
		a.partial = s->partial;
		a.tickets = s->tickets;
		a.out = s->logits + size_t(b0) * V;
		TG_TRY(launch_mv(a, PRO_RESNORM, EPI_SCALE, st));
	}
	return TG_OK;
}


int batched_setup(tg_state *s);
int enqueue_decode_batched(tg_state *s, bool with_lm_head);


int enqueue_decode_all(tg_state *s) {
	if (s->batched_ok) return enqueue_decode_batched(s, true);
	for (int b0 = 0; b0 < s->B; b0 += MV_MAX_B) TG_TRY(enqueue_decode_chunk(s, b0, std::min(MV_MAX_B, s->B - b0)));
	return TG_OK;
}

int enqueue_decode_step(tg_state *s) {
	// The first step of a state runs eagerly so that lazy module loading and
	// cudaFuncSetAttribute happen outside stream capture; the graph is captured
	// on the second step and replayed from then on.
	if (!s->use_graph || !s->warmed) {
		s->warmed = true;
		return enqueue_decode_all(s);
	}
	if (!s->graph) {
		cudaGraph_t g = nullptr;
		long long before = g_launches.load();
		TG_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
		int rc = enqueue_decode_all(s);
		cudaError_t e = cudaStreamEndCapture(s->stream, &g);
		s->graph_launches = int(g_launches.load() - before);
		g_launches.store(before);
		if (rc != TG_OK) {
			if (g) cudaGraphDestroy(g);
			return rc;
		}
		if (e != cudaSuccess) return fail(TG_ECUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
		e = cudaGraphInstantiate(&s->graph, g, 0);
		cudaGraphDestroy(g);
		if (e != cudaSuccess) return fail(TG_ECUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
	}
	TG_CUDA(cudaGraphLaunch(s->graph, s->stream));
	count_launch(s->graph_launches);
	return TG_OK;
}

// ------------------------------------------------------------- persistent kernel set-up
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled get_encode_fn() {
	static PFN_encodeTiled fn = nullptr;
	if (!fn) {
		void *p = nullptr;
		cudaDriverEntryPointQueryResult q;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
		    q == cudaDriverEntryPointSuccess)
			fn = reinterpret_cast<PFN_encodeTiled>(p);
	}
	return fn;
}

// 2-D uint8 map over a row-major [K, N] int8 matrix; box = TN bytes x box_rows rows, no swizzle
int make_tmap(CUtensorMap *out, const int8_t *base, int K, int N, int TN, int box_rows, int ld = 0) {
	PFN_encodeTiled enc = get_encode_fn();
	if (!enc) return fail(TG_ECUDA, "cuTensorMapEncodeTiled entry point not available");
	cuuint64_t gdim[2] = {cuuint64_t(N), cuuint64_t(K)};
	cuuint64_t gstride[1] = {cuuint64_t(ld > 0 ? ld : N)};
	cuuint32_t box[2] = {cuuint32_t(TN), cuuint32_t(box_rows)};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(base), gdim, gstride, box, estr,
	                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
	                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) return fail(TG_ECUDA, "cuTensorMapEncodeTiled failed: " + std::to_string(int(r)));
	return TG_OK;
}

int largest_box_rows(int kc) {
	for (int r = std::min(kc, 256); r >= 1; r--)
		if (kc % r == 0) return r;
	return 1;
}

// thread-mapping constants of a phase: x / d == __umulhi(x, ceil(2^32 / d)) for x * d < 2^32
void mg_fill_mapping(MgPhase *ph) {
	ph->rstep = MG_THREADS / ph->segs;
	ph->m_segs = unsigned((0x100000000ull + ph->segs - 1) / ph->segs);
	ph->m_rstep = unsigned((0x100000000ull + ph->rstep - 1) / ph->rstep);
}

// Choose the tile width and K-split of one phase so that as many of the G CTAs
// as possible get exactly one unit. n_cols lists the matrices that share the
// phase's column tiling (Q,K,V) — a tile never straddles two of them.
bool plan_phase(MgPhase *out, int K, const std::vector<int> &n_cols, int nmat, bool allow_split, int G, int max_bytes) {
	const int tns[] = {128, 96, 64, 48, 32, 16};
	long best_score = -1;
	for (int TN : tns) {
		const int segs = TN / 16;
		if (MG_THREADS % segs) continue;
		bool ok = true;
		int ntiles = 0;
		for (int n : n_cols) {
			if (n % TN) ok = false;
			ntiles += n / TN;
		}
		if (!ok || ntiles > G) continue;
		for (int ns = 1; ns <= (allow_split ? 64 : 1); ns++) {
			if (K % ns) continue;
			const int kc = K / ns;
			if (kc % 8) continue;
			const int units = ntiles * ns;
			if (units > G) break;
			const long bytes = long(nmat) * TN * kc;
			if (bytes > max_bytes) continue;
			// as many busy SMs as possible; then few K-splits (every CTA re-reads all split partial sums in
			// its norm prologue); 16-column tiles are avoided (measured: O projection as 16 x 512 x 2 splits
			// instead of 32 x 256 x 4 doubles the attention-merge rows per CTA and loses 2.5 %)
			long score = long(units) * 1000 - ns * env_int("TG_MEGA_SPLIT_COST", 40) - (TN < 32 ? 2000 : 0);
			if (score > best_score) {
				best_score = score;
				const int br = largest_box_rows(kc);
				*out = MgPhase{TN, segs, ns, kc, br, kc / br, ntiles, units, int(bytes), 0, 0u, 0u};
				mg_fill_mapping(out);
			}
		}
	}
	return best_score >= 0;
}

int mega_setup(tg_state *s) {
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab, L = c.n_layers;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	int dev = m->device, coop = 0, smem_max = 0;
	TG_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
	TG_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
	if (!coop) return fail(TG_ECUDA, "device lacks cooperative launch");
	const int G = env_int("TG_MEGA_GRID", g_num_sms);
	MgArgs &a = s->mega;
	a = MgArgs{};
	// (the CTAs that idle through the attention phase wipe the hand-off arena: at least 8 must remain)
	if (G < 16) return fail(TG_ESHAPE, "persistent kernel: grid too small");
	a.att_local = std::min(std::min(env_int("TG_MEGA_ATT_LOCAL", 32), MG_MAX_ATT), G - 8);
	a.att_global = std::min(std::min(env_int("TG_MEGA_ATT_GLOBAL", 32), MG_MAX_ATT), G - 8);
	const int budget = smem_max - 40 * 1024;  // room for h, xs, reduction scratch, attention scratch, static shared
	if (!plan_phase(&a.A, D, {qd, kd, kd}, 1, true, G, budget / 8) || !plan_phase(&a.C, qd, {D}, 1, true, G, budget / 8) ||
	    !plan_phase(&a.Dp, D, {I}, 2, false, G, budget) || !plan_phase(&a.E, I, {D}, 1, true, G, budget / 2))
		return fail(TG_ESHAPE, "no phase plan fits");
	a.LM = MgPhase{MG_LM_TN, MG_LM_TN / 16, 1, D, largest_box_rows(D), D / largest_box_rows(D), V / MG_LM_TN, V / MG_LM_TN, 0, 0, 0u, 0u};
	mg_fill_mapping(&a.LM);
	a.lm_bps = (a.LM.nboxes % 2 == 0) ? 2 : 1;  // TMA boxes per ring stage
	const int ring = MG_LM_STAGES * a.LM.TN * a.LM.box_rows * a.lm_bps;
	auto up = [](int v) { return (v + 1023) & ~1023; };
	int off = 0;
	a.off_A = off;
	off = up(off + a.A.bytes);
	a.off_C = off;
	off = up(off + a.C.bytes);
	a.off_D = off;
	a.off_E = off + a.Dp.bytes;  // contiguous with D: the lm_head ring overlays both
	off = up(off + std::max(a.Dp.bytes + a.E.bytes, std::max(ring, 8192 * 4)));
	a.off_h = off;
	off = up(off + D * 4);
	a.off_xs = off;
	off = up(off + std::max(std::max(D, a.E.kc), std::max(a.A.kc, a.C.kc)) * 4);
	a.off_red = off;
	off = up(off + std::max(MG_NWARPS * AT_HD * 4, std::max((qd + 2 * kd) * 4, MG_NWARPS * 128 * 4)));
	a.off_att = off;
	off = up(off + (AT_NH + 2) * AT_HD * 4);
	a.smem_total = off + 1024;
	if (a.smem_total + 8 * 1024 > smem_max) return fail(TG_ESHAPE, "persistent kernel does not fit in shared memory");
	if (L > MG_MAX_LAYERS || D > 3 * MG_THREADS || a.A.nsplit > 8 || std::max(a.att_local, a.att_global) * 8 * 4 > (AT_NH + 2) * AT_HD * 4)
		return fail(TG_ESHAPE, "persistent kernel limits exceeded");
	if ((a.Dp.bytes % 16) || (a.off_E % 128)) return fail(TG_ESHAPE, "region alignment");

	// one tensor map (lm_head); the layer weights come from the re-tiled copy
	std::vector<CUtensorMap> maps(1);
	std::vector<MgLayer> lys(L);
	for (int l = 0; l < L; l++) {
		const LayerW &w = m->layers[l];
		MgLayer &ly = lys[l];
		ly.sq = w.Q.s;
		ly.sk = w.K.s;
		ly.sv = w.V.s;
		ly.so = w.O.s;
		ly.su = w.U.s;
		ly.sg = w.G.s;
		ly.sd = w.Dn.s;
		ly.rmsq = w.rmsq;
		ly.rmsk = w.rmsk;
		ly.attn_pre = w.attn_pre;
		ly.attn_post = w.attn_post;
		ly.mlp_pre = w.mlp_pre;
		ly.mlp_post = w.mlp_post;
		ly.kcache = s->kcache[l];
		ly.vcache = s->vcache[l];
		ly.slots = s->slots[l];
		ly.is_local = w.is_local ? 1 : 0;
	}
	TG_TRY(make_tmap(&maps[0], m->lm_head.q, D, V, a.LM.TN, a.LM.box_rows));
	a.tm_lm = 0;
	a.tl_A = 0;
	a.tl_C = a.tl_A + size_t(a.A.units) * a.A.bytes;
	a.tl_D = a.tl_C + size_t(a.C.units) * a.C.bytes;
	a.tl_E = a.tl_D + size_t(a.Dp.units) * a.Dp.bytes;
	a.tl_layer = a.tl_E + size_t(a.E.units) * a.E.bytes;
	TG_CUDA(cudaMalloc(&s->d_tmaps, maps.size() * sizeof(CUtensorMap)));
	TG_CUDA(cudaMemcpy(s->d_tmaps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
	TG_CUDA(cudaMalloc(&s->d_layers, lys.size() * sizeof(MgLayer)));
	TG_CUDA(cudaMemcpy(s->d_layers, lys.data(), lys.size() * sizeof(MgLayer), cudaMemcpyHostToDevice));
	auto allocz = [&](void **p, size_t bytes) -> int {
		TG_CUDA(cudaMalloc(p, bytes));
		TG_CUDA(cudaMemset(*p, 0, bytes));
		return TG_OK;
	};
	// hand-off arena (two copies) and the double-buffered down-projection partial sums
	auto up4 = [](int n) { return (n + 3) & ~3; };
	a.ll_pA = 0;
	a.ll_att = a.ll_pA + up4(a.A.nsplit * (qd + 2 * kd));
	a.ll_pC = a.ll_att + up4(MG_MAX_ATT * (AT_NH * AT_HD + 8));
	a.ll_act = a.ll_pC + up4(a.C.nsplit * D);
	a.ll_stride = a.ll_act + up4(I);
	s->mg_ll_bytes = size_t(2) * a.ll_stride * 4;
	TG_CUDA(cudaMalloc(&s->mg_ll, s->mg_ll_bytes));
	TG_CUDA(cudaMemset(s->mg_ll, 0xFF, s->mg_ll_bytes));
	a.pe_stride = a.E.nsplit * D + ((G - a.E.units + 3) & ~3) + 4;
	TG_TRY(allocz((void **)&s->mg_pe, size_t(2) * a.pe_stride * sizeof(uint2)));
	TG_TRY(allocz((void **)&s->mg_samp_f, size_t(3) * G * 4));
	TG_TRY(allocz((void **)&s->mg_samp_i, size_t(G + 8) * 4));
	TG_TRY(allocz((void **)&s->mg_bar, 64));
	a.tmaps = s->d_tmaps;
	a.layers = s->d_layers;
	a.L = L;
	a.D = D;
	a.I = I;
	a.V = V;
	a.QD = qd;
	a.KD = kd;
	a.lm_scale = m->lm_head.s;
	a.final_norm = m->final_norm;
	a.wte = m->wte;
	a.wte_s = m->wte_s;
	a.sqrtD = float(std::sqrt(double(D)));
	a.ll = s->mg_ll;
	a.pe = s->mg_pe;
	a.logits = s->logits;
	TG_TRY(allocz((void **)&s->mg_probs, size_t(V) * 4));
	a.probs = s->mg_probs;
	{
		const int region_floats = (a.off_h - a.off_D) / 4;
		a.samp_ch = std::max(3072, std::min(region_floats, 24576) / 3072 * 3072);
		if (a.samp_ch > region_floats) return fail(TG_ESHAPE, "sampler staging does not fit the weight ring");
	}
	a.samp_f = s->mg_samp_f;
	a.samp_i = s->mg_samp_i;
	a.xnorm_out = s->xnorm;
	a.bar = s->mg_bar;
	a.err = s->err_flag;
	a.tok = s->tok;
	a.next_pos = s->next_pos;
	a.ring_base = s->ring_base;
	a.log_count = s->log_count;
	a.randf_count = s->randf_count;
	TG_CUDA(cudaFuncSetAttribute(mega_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, a.smem_total));
	int per_sm = 0;
	TG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mega_decode_kernel, MG_THREADS, a.smem_total));
	if (per_sm < 1 || G > per_sm * g_num_sms) return fail(TG_ESHAPE, "persistent kernel cannot be co-resident");
	s->mega_grid = G;
	s->mega_smem = a.smem_total;
	s->mega_ok = true;
	if (env_int("TG_MEGA_VERBOSE", 0))
		fprintf(stderr,
		        "[tg] mega plan: A TN%d x%d kc%d (%d units)  C TN%d x%d kc%d (%d)  D TN%d (%d)  E TN%d x%d kc%d (%d)  "
		        "LM box %d  smem %d B  grid %d\n",
		        a.A.TN, a.A.nsplit, a.A.kc, a.A.units, a.C.TN, a.C.nsplit, a.C.kc, a.C.units, a.Dp.TN, a.Dp.units, a.E.TN,
		        a.E.nsplit, a.E.kc, a.E.units, a.LM.box_rows, a.smem_total, G);
	return TG_OK;
}

// Build (or refresh after a reload of the weights) the model's copy of the layer weights in unit
// order: for every layer the units of phase A (q|k|v column tiles x K-splits), C (O projection),
// D (up tile followed by the gate tile of the same columns) and E (down projection), each unit a
// contiguous [rows][TN] block, so that a CTA fetches its unit with sequential bulk copies.
int ensure_decode_tiles(tg_state *s) {
	tg_model *m = s->m;
	const MgArgs &a = s->mega;
	const tg_config &c = m->cfg;
	const int L = c.n_layers, D = c.hidden_size, I = c.intermediate_size;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	const int key[12] = {a.A.TN, a.A.nsplit, a.C.TN, a.C.nsplit, a.Dp.TN, a.Dp.nsplit, a.E.TN, a.E.nsplit, s->mega_grid, L, D, I};
	if (m->dec_tiled && m->dec_tiled_version == m->weights_version && std::memcmp(key, m->dec_tiled_key, sizeof key) == 0)
		return TG_OK;
	const size_t bytes = a.tl_layer * L;
	if (m->dec_tiled_bytes != bytes) {
		cudaFree(m->dec_tiled);
		m->dec_tiled = nullptr;
		TG_CUDA(cudaMalloc(&m->dec_tiled, bytes));
		m->dec_tiled_bytes = bytes;
	}
	cudaStream_t st = s->stream;
	auto run = [&](int8_t *dst, const QW &w, const MgPhase &ph, int ntiles_total, int tile0, size_t unit_stride, size_t dst_off) {
		const int ntiles_mat = w.N / ph.TN;
		retile_kernel<<<4 * g_num_sms, 256, 0, st>>>(dst, w.q, w.N, ph.TN, ph.kc, ph.nsplit, ntiles_total, tile0, ntiles_mat,
		                                             unit_stride, dst_off);
		count_launch();
	};
	for (int l = 0; l < L; l++) {
		const LayerW &w = m->layers[l];
		int8_t *base = m->dec_tiled + size_t(l) * a.tl_layer;
		run(base + a.tl_A, w.Q, a.A, a.A.ntiles, 0, a.A.bytes, 0);
		run(base + a.tl_A, w.K, a.A, a.A.ntiles, qd / a.A.TN, a.A.bytes, 0);
		run(base + a.tl_A, w.V, a.A, a.A.ntiles, (qd + kd) / a.A.TN, a.A.bytes, 0);
		run(base + a.tl_C, w.O, a.C, a.C.ntiles, 0, a.C.bytes, 0);
		run(base + a.tl_D, w.U, a.Dp, a.Dp.ntiles, 0, a.Dp.bytes, 0);
		run(base + a.tl_D, w.G, a.Dp, a.Dp.ntiles, 0, a.Dp.bytes, size_t(a.Dp.TN) * D);
		run(base + a.tl_E, w.Dn, a.E, a.E.ntiles, 0, a.E.bytes, 0);
	}
	TG_TRY(check_launch("retile"));
	std::memcpy(m->dec_tiled_key, key, sizeof key);
	m->dec_tiled_version = m->weights_version;
	return TG_OK;
}


// ---------------------------------------------------------------- dp4a persistent decode kernel
// Plan of one phase: column groups per unit, K-splits across CTAs and warps per group, chosen by an
// estimate of the phase's time in clocks: the tile product (measured: about 650 clk fixed + 1 clk per
// 55 bytes, 65 with two matrices that share the activations) plus the bytes the phase makes CTAs poll
// (measured: about 76 clk per KB and CTA). `poll_kb(nsplit)` gives those KB for a split.
template <class F>
bool ps_plan(PsPhase *out, int K, int N, int nmat, int G, int max_bytes, const std::vector<int> &splits,
             const std::vector<int> &col_blocks, int max_nq, F poll_kb) {
	double best = 1e30;
	for (int ns : splits) {
		if ((K / 4) % ns) continue;
		const int nq = K / 4 / ns;
		if (nq > max_nq) continue;
		for (int ng = 1; ng <= PS_NW; ng++) {
			bool ok = (N / 4) % ng == 0;
			for (int cb : col_blocks) ok = ok && (cb / 4) % ng == 0;  // a tile never straddles two matrices
			if (!ok) continue;
			const int ntiles = N / 4 / ng, units = ntiles * ns;
			if (units > G) continue;
			const int bytes = nmat * ng * nq * 16;
			if (bytes > max_bytes) continue;
			const int kp = std::max(1, std::min(PS_NW / ng, (nq + 31) / 32));
			const double cost = 650.0 + double(bytes) / (nmat == 2 ? 65.0 : 55.0) + 76.0 * poll_kb(ns);
			if (cost < best) {
				best = cost;
				*out = PsPhase{ng, nq, ns, ntiles, units, kp, (nq + kp - 1) / kp, bytes, 0};
			}
		}
	}
	return best < 1e30;
}

int persist_setup(tg_state *s) {
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab, L = c.n_layers;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	int smem_max = 0;
	TG_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->device));
	const int G = s->mega_grid;
	PsArgs &a = s->ps;
	a = PsArgs{};
	if (c.n_head != AT_NH || c.head_dim != AT_HD || c.n_kv != 1 || D % 4 || I % 4 || D > 4 * PS_THREADS || L > PS_MAX_LAYERS)
		return fail(TG_ESHAPE, "persistent kernel: unsupported shape");
	const int budget = smem_max - 48 * 1024;
	const double dkb = D * 4 / 1024.0;
	const int csplit = env_int("TG_PS_C_SPLIT", 0), esplit = env_int("TG_PS_E_SPLIT", 0);
	if (!ps_plan(&a.A, D, qd + 2 * kd, 1, G, budget / 6, {1, 2, 3, 4}, {qd, kd}, 1 << 20,
	             [&](int ns) { return 3.0 * ns; }) ||
	    !ps_plan(&a.C, qd, D, 1, G, budget / 8, csplit ? std::vector<int>{csplit} : std::vector<int>{1, 2, 4}, {}, 1 << 20,
	             [&](int ns) { return 8.0 * (AT_NH / ns) + dkb * ns; }) ||
	    !ps_plan(&a.Dp, D, I, 2, G, budget, {1}, {}, 1 << 20, [&](int) { return 0.0; }) ||
	    !ps_plan(&a.E, I, D, 1, G, budget / 2, esplit ? std::vector<int>{esplit} : std::vector<int>{1, 2, 3, 4, 6, 8}, {},
	             5 * PS_THREADS, [&](int ns) { return I * 4 / 1024.0 / ns + dkb * ns; }))
		return fail(TG_ESHAPE, "persistent kernel: no phase plan fits");
	a.A.cta0 = G - a.A.units;  // the attention CTAs (low indices) hold no Q|K|V unit where possible
	// cache chunks per head; at least 8 CTAs must stay out of the attention phase (they wipe the hand-off arena)
	const int chmax = std::max(1, std::min(PS_MAX_CH, (G - 8) / AT_NH));
	a.nch_local = std::min(chmax, env_int("TG_PS_NCH_LOCAL", 8));
	a.nch_mid = std::min(chmax, env_int("TG_PS_NCH_MID", 16));
	a.nch_long = std::min(chmax, env_int("TG_PS_NCH_LONG", 32));
	const int npres = G - a.E.units;
	if (D / 4 + npres > PS_THREADS || G < 16) return fail(TG_ESHAPE, "persistent kernel: grid too small for the down-projection plan");
	// lm_head: tiles of 24 column groups (two per warp); ring stages of at most ~40 KB
	a.lm_groups = 2 * PS_NW;
	a.lm_cq = D / 4;
	for (int n = 1; n <= 16; n++)
		if ((D / 4) % n == 0 && a.lm_groups * (D / 4 / n) * 16 <= 40 * 1024) {
			a.lm_cq = D / 4 / n;
			break;
		}
	a.lm_nchunk = D / 4 / a.lm_cq;
	a.lm_ntiles = (V + a.lm_groups * 4 - 1) / (a.lm_groups * 4);
	a.lm_stage_bytes = a.lm_groups * a.lm_cq * 16;
	auto up = [](int v) { return (v + 127) & ~127; };
	int off = 0;
	a.off_A = off;
	off = up(off + a.A.bytes);
	a.off_C = off;
	off = up(off + a.C.bytes);
	a.off_D = off;
	a.off_E = off + a.Dp.bytes;  // contiguous with the up/gate region: the lm_head ring and the sampler staging overlay both
	const int region = std::max(std::max(a.Dp.bytes + a.E.bytes, 3072 * 4), std::min(3 * a.lm_stage_bytes, smem_max / 2));
	off = up(off + region);
	a.lm_stages = std::min(8, region / a.lm_stage_bytes);
	if (a.lm_stages < 2) return fail(TG_ESHAPE, "persistent kernel: lm_head ring does not fit");
	a.off_h = off;
	off = up(off + D * 4);
	a.xd_words = std::max(std::max(D / 4, a.E.nq), qd / 4);
	a.off_xd = off;
	off = up(off + 3 * a.xd_words * 4);
	a.off_att = off;
	off = up(off + (PS_NW * AT_HD + 4 * AT_HD) * 4);
	a.smem_total = off + 128;
	{
		const int region_floats = region / 4;
		a.samp_ch = std::min(region_floats, 24576) / 3072 * 3072;
		if (a.samp_ch < 3072) return fail(TG_ESHAPE, "persistent kernel: sampler staging does not fit");
	}
	cudaFuncAttributes fa{};
	TG_CUDA(cudaFuncGetAttributes(&fa, decode_persist_kernel<true>));
	if (a.smem_total + int(fa.sharedSizeBytes) > smem_max) return fail(TG_ESHAPE, "persistent kernel does not fit in shared memory");

	std::vector<PsLayer> lys(L);
	for (int l = 0; l < L; l++) {
		const LayerW &w = m->layers[l];
		PsLayer &ly = lys[l];
		ly.sq = w.Q.s;
		ly.sk = w.K.s;
		ly.sv = w.V.s;
		ly.so = w.O.s;
		ly.su = w.U.s;
		ly.sg = w.G.s;
		ly.sd = w.Dn.s;
		ly.rmsq = w.rmsq;
		ly.rmsk = w.rmsk;
		ly.attn_pre = w.attn_pre;
		ly.attn_post = w.attn_post;
		ly.mlp_pre = w.mlp_pre;
		ly.mlp_post = w.mlp_post;
		ly.kcache = s->kcache[l];
		ly.vcache = s->vcache[l];
		ly.slots = s->slots[l];
		ly.is_local = w.is_local ? 1 : 0;
	}
	TG_CUDA(cudaMalloc(&s->d_pslayers, lys.size() * sizeof(PsLayer)));
	TG_CUDA(cudaMemcpy(s->d_pslayers, lys.data(), lys.size() * sizeof(PsLayer), cudaMemcpyHostToDevice));
	a.tl_A = 0;
	a.tl_C = a.tl_A + size_t(a.A.units) * a.A.bytes;
	a.tl_D = a.tl_C + size_t(a.C.units) * a.C.bytes;
	a.tl_E = a.tl_D + size_t(a.Dp.units) * a.Dp.bytes;
	a.tl_layer = a.tl_E + size_t(a.E.units) * a.E.bytes;
	auto up4 = [](int n) { return (n + 3) & ~3; };
	a.ll_qkv = 0;
	a.ll_att = up4(qd + 2 * kd);
	a.ll_op = a.ll_att + AT_NH * PS_MAX_CH * PS_ATT_ROW;
	a.ll_act = a.ll_op + a.C.nsplit * D;
	a.ll_dn = a.ll_act + I;
	a.ll_pres = a.ll_dn + a.E.nsplit * D;
	a.ll_stride = up4(a.ll_pres + npres + 4);
	s->ps_ll_bytes = size_t(3) * a.ll_stride * 4;
	TG_CUDA(cudaMalloc(&s->ps_ll, s->ps_ll_bytes));
	TG_CUDA(cudaMemset(s->ps_ll, 0xFF, s->ps_ll_bytes));
	a.layers = s->d_pslayers;
	a.L = L;
	a.D = D;
	a.I = I;
	a.V = V;
	a.QD = qd;
	a.KD = kd;
	a.lm_scale = m->lm_head.s;
	a.final_norm = m->final_norm;
	a.wte = m->wte;
	a.wte_s = m->wte_s;
	a.sqrtD = float(std::sqrt(double(D)));
	a.ll = s->ps_ll;
	a.logits = s->logits;
	a.probs = s->mg_probs;
	a.samp_f = s->mg_samp_f;
	a.samp_i = s->mg_samp_i;
	a.xnorm_out = s->xnorm;
	a.bar = s->mg_bar;
	a.err = s->err_flag;
	a.tok = s->tok;
	a.next_pos = s->next_pos;
	a.ring_base = s->ring_base;
	a.log_count = s->log_count;
	a.randf_count = s->randf_count;
	TG_CUDA(cudaFuncSetAttribute(decode_persist_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, a.smem_total));
	TG_CUDA(cudaFuncSetAttribute(decode_persist_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, a.smem_total));
	int per_sm = 0;
	TG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persist_kernel<true>, PS_THREADS, a.smem_total));
	if (per_sm < 1 || G > per_sm * g_num_sms) return fail(TG_ESHAPE, "persistent kernel cannot be co-resident");
	s->ps_ok = true;
	if (env_int("TG_MEGA_VERBOSE", 0))
		fprintf(stderr,
		        "[tg] persist plan: A %dg x%d nq%d kp%d (%d units)  C %dg x%d nq%d kp%d (%d)  D %dg nq%d kp%d (%d)  E %dg x%d nq%d kp%d (%d)  "
		        "lm cq %d x%d stages %d  smem %d + %d B  grid %d\n",
		        a.A.ngroups, a.A.nsplit, a.A.nq, a.A.kp, a.A.units, a.C.ngroups, a.C.nsplit, a.C.nq, a.C.kp, a.C.units, a.Dp.ngroups,
		        a.Dp.nq, a.Dp.kp, a.Dp.units, a.E.ngroups, a.E.nsplit, a.E.nq, a.E.kp, a.E.units, a.lm_cq, a.lm_nchunk, a.lm_stages,
		        a.smem_total, int(fa.sharedSizeBytes), G);
	return TG_OK;
}

// Build (or refresh after a reload of the weights) the model's copies in the kernel's unit order:
// per layer the units of phase A (q|k|v), C (O projection), D (up pieces followed by the gate pieces of
// the same columns) and E (down projection), and the lm_head in ring-stage order.
int ensure_persist_tiles(tg_state *s) {
	tg_model *m = s->m;
	const PsArgs &a = s->ps;
	const tg_config &c = m->cfg;
	const int L = c.n_layers, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	const int key[20] = {a.A.ngroups, a.A.nsplit, a.A.nq, a.C.ngroups, a.C.nsplit, a.C.nq, a.Dp.ngroups, a.Dp.nq, a.E.ngroups, a.E.nsplit,
	                     a.E.nq,      a.lm_groups, a.lm_cq, a.lm_ntiles, L, a.D, a.I, V, 0, 0};
	if (m->ps_tiled && m->ps_tiled_version == m->weights_version && std::memcmp(key, m->ps_tiled_key, sizeof key) == 0) return TG_OK;
	const size_t bytes = a.tl_layer * L;
	const size_t lm_bytes = size_t(a.lm_ntiles) * a.lm_nchunk * a.lm_stage_bytes;
	if (m->ps_tiled_bytes != bytes) {
		cudaFree(m->ps_tiled);
		m->ps_tiled = nullptr;
		TG_CUDA(cudaMalloc(&m->ps_tiled, bytes));
		m->ps_tiled_bytes = bytes;
	}
	if (m->ps_lm_bytes != lm_bytes) {
		cudaFree(m->ps_lm);
		m->ps_lm = nullptr;
		TG_CUDA(cudaMalloc(&m->ps_lm, lm_bytes));
		m->ps_lm_bytes = lm_bytes;
	}
	cudaStream_t st = s->stream;
	auto run = [&](int8_t *dst, const QW &w, const PsPhase &ph, int tile0, size_t dst_off) {
		retile_quads_kernel<<<4 * g_num_sms, 256, 0, st>>>(dst, w.q, w.N, ph.ngroups, ph.nq, ph.nsplit, ph.ntiles, tile0,
		                                                   w.N / 4 / ph.ngroups, size_t(ph.bytes), dst_off);
		count_launch();
	};
	for (int l = 0; l < L; l++) {
		const LayerW &w = m->layers[l];
		int8_t *base = m->ps_tiled + size_t(l) * a.tl_layer;
		run(base + a.tl_A, w.Q, a.A, 0, 0);
		run(base + a.tl_A, w.K, a.A, qd / 4 / a.A.ngroups, 0);
		run(base + a.tl_A, w.V, a.A, (qd + kd) / 4 / a.A.ngroups, 0);
		run(base + a.tl_C, w.O, a.C, 0, 0);
		run(base + a.tl_D, w.U, a.Dp, 0, 0);
		run(base + a.tl_D, w.G, a.Dp, 0, size_t(a.Dp.ngroups) * a.Dp.nq * 16);
		run(base + a.tl_E, w.Dn, a.E, 0, 0);
	}
	retile_lm_kernel<<<8 * g_num_sms, 256, 0, st>>>(m->ps_lm, m->lm_head.q, V, a.lm_groups, a.lm_cq, a.lm_nchunk, a.lm_ntiles);
	count_launch();
	TG_TRY(check_launch("retile"));
	std::memcpy(m->ps_tiled_key, key, sizeof key);
	m->ps_tiled_version = m->weights_version;
	return TG_OK;
}

int persist_launch(tg_state *s, int n_steps, int sampler, float minp, float temp, bool log_tokens, const int *force_ids = nullptr) {
	tg_model *m = s->m;
	TG_TRY(ensure_persist_tiles(s));
	PsArgs a = s->ps;
	a.tiled = m->ps_tiled;
	a.lm_tiled = m->ps_lm;
	a.rope[0][0] = m->rope[0][0];
	a.rope[0][1] = m->rope[0][1];
	a.rope[1][0] = m->rope[1][0];
	a.rope[1][1] = m->rope[1][1];
	a.lut = make_lut(m);
	a.n_steps = n_steps;
	a.sampler = sampler;
	a.force_ids = force_ids;
	a.minp = minp;
	a.temp = temp;
	a.randf = s->lean_randf ? s->randf_blk : s->randf;
	a.randf_cap = s->lean_randf ? STEP_RANDF : s->randf_cap;
	s->lean_randf = false;
	a.tok_log = log_tokens ? s->tok_log : nullptr;
	a.log_cap = s->log_cap;
	a.dbg = s->mg_dbg;
	a.dbg_cap = s->mg_dbg ? 4096 : 0;
	a.dbg_cta = std::min(std::max(env_int("TG_MEGA_DBG_CTA", 0), 0), s->mega_grid - 1);
	a.wait_clocks = (long long)(std::max(1, env_int("TG_PS_WAIT_MS", 100))) * 2000000ll;  // ~2 GHz
	a.fault_cta = env_int("TG_PS_WITHHOLD_CTA", -1);
	a.e_wq = (a.E.nq + PS_NW - 1) / PS_NW;
	a.e_rows = (env_int("TG_PS_E_ROWS", 0) && a.E.ngroups <= 4 && a.e_wq <= 96) ? 1 : 0;
	a.poll_ns = std::max(0, env_int("TG_PS_POLL_NS", 20));
	a.sched = env_int("TG_PS_SCHED", 0);
	a.gt = (s->mg_dbg && env_int("TG_PS_GT", 0)) ? s->mg_dbg + 2048 : nullptr;  // (the stamp recorder uses < 600 entries)
	// Every word of the hand-off arena copy 0 starts as "empty" (all ones) and the barrier counter at
	// bar_base: a launch that ran through leaves both that way. After an error (or before the first
	// launch) they are set here.
	if (!s->ps_clean) {
		TG_CUDA(cudaMemsetAsync(s->ps_ll, 0xFF, s->ps_ll_bytes, s->stream));
		TG_CUDA(cudaMemsetAsync(s->mg_bar, 0, 4, s->stream));
		s->ps_bar_base = 0;
		s->ps_clean = true;
	}
	a.bar_base = s->ps_bar_base;
	// TG_PS_BEACON=1: every warp leaves progress marks in mapped host memory; if the launch has not finished
	// after two seconds the marks are printed (where each CTA's slowest and fastest warp stand)
	static int *beacon_host = nullptr, *beacon_dev = nullptr;
	const bool beacon = env_int("TG_PS_BEACON", 0) != 0;
	if (beacon && !beacon_host) {
		TG_CUDA(cudaHostAlloc(&beacon_host, 1024 * 16 * 4, cudaHostAllocMapped));
		TG_CUDA(cudaHostGetDevicePointer(&beacon_dev, beacon_host, 0));
	}
	if (beacon) std::memset(beacon_host, 0, 1024 * 16 * 4);
	a.beacon = beacon ? beacon_dev : nullptr;
	void *params[] = {&a};
	// the instrumented instantiation runs only while the phase-clock recorder or the progress marks are armed
	const void *fn = (a.dbg || a.beacon) ? (const void *)decode_persist_kernel<true> : (const void *)decode_persist_kernel<false>;
	TG_CUDA(cudaLaunchCooperativeKernel(fn, dim3(s->mega_grid), dim3(PS_THREADS), params, size_t(a.smem_total), s->stream));
	count_launch();
	TG_TRY(check_launch("decode_persist"));
	// grid barriers per token: logits complete / the arg-max, and two more for min-p (denominator, drawn index)
	s->ps_bar_base += unsigned(n_steps) * unsigned(sampler == 2 ? 3 : 1) * unsigned(s->mega_grid);
	if (beacon) {
		for (int ms = 0; ms < 2000 && cudaStreamQuery(s->stream) == cudaErrorNotReady; ms++) {
			struct timespec ts = {0, 1000000};
			nanosleep(&ts, nullptr);
		}
		if (cudaStreamQuery(s->stream) == cudaErrorNotReady) {
			fprintf(stderr, "[tg] persistent kernel still running after 2 s; marks (layer count : phase mark) per CTA, min..max over its warps:\n");
			for (int c = 0; c < s->mega_grid; c++) {
				int lo = INT_MAX, hi = 0;
				for (int w = 0; w < PS_NW; w++) {
					lo = std::min(lo, beacon_host[c * 16 + w]);
					hi = std::max(hi, beacon_host[c * 16 + w]);
				}
				fprintf(stderr, " %d=%d:%02x..%d:%02x", c, lo >> 8, lo & 0xFF, hi >> 8, hi & 0xFF);
				if (c % 8 == 7) fprintf(stderr, "\n");
			}
			fprintf(stderr, "\n");
			fflush(stderr);
		}
		cudaGetLastError();
	}
	return TG_OK;
}

// one cooperative launch: n_steps tokens; sampler 0 none / 1 argmax / 2 min-p
int mega_launch(tg_state *s, int n_steps, int sampler, float minp, float temp, bool log_tokens) {
	if (s->ps_ok) return persist_launch(s, n_steps, sampler, minp, temp, log_tokens);
	tg_model *m = s->m;
	TG_TRY(ensure_decode_tiles(s));
	MgArgs a = s->mega;
	a.tiled = m->dec_tiled;
	a.rope[0][0] = m->rope[0][0];
	a.rope[0][1] = m->rope[0][1];
	a.rope[1][0] = m->rope[1][0];
	a.rope[1][1] = m->rope[1][1];
	a.lut = make_lut(m);
	a.n_steps = n_steps;
	a.sampler = sampler;
	a.minp = minp;
	a.temp = temp;
	a.randf = s->randf;
	a.randf_cap = s->randf_cap;
	a.tok_log = log_tokens ? s->tok_log : nullptr;
	a.log_cap = s->log_cap;
	a.seq0 = s->mg_seq;
	s->mg_seq += unsigned(n_steps) * unsigned(m->cfg.n_layers);
	// CTAs per global-attention layer follow the context: 32 up to ~1K positions, 64 beyond (measured at 16K
	// positions: 937 -> 1049 tok/s; at 200-700 positions 64 is no gain). TG_MEGA_ATT_GLOBAL fixes the number.
	if (!std::getenv("TG_MEGA_ATT_GLOBAL") && s->host_pos[0] >= 1024) a.att_global = std::min(MG_MAX_ATT, s->mega_grid - 8);
	// every word of the hand-off arena starts as "empty" (all ones)
	TG_CUDA(cudaMemsetAsync(s->mg_ll, 0xFF, s->mg_ll_bytes, s->stream));
	a.dbg = s->mg_dbg;
	a.dbg_cap = s->mg_dbg ? 4096 : 0;
	a.sched = env_int("TG_MEGA_SCHED", 1);
	a.dbg_cta = std::min(std::max(env_int("TG_MEGA_DBG_CTA", 0), 0), s->mega_grid - 1);
	TG_CUDA(cudaMemsetAsync(s->mg_bar, 0, 4, s->stream));
	void *params[] = {&a};
	TG_CUDA(cudaLaunchCooperativeKernel((void *)mega_decode_kernel, dim3(s->mega_grid), dim3(MG_THREADS), params,
	                                    s->mega_smem, s->stream));
	count_launch();
	return check_launch("mega_decode");
}

SampleArgs sample_args(tg_state *s, float minp, float temp, bool log_tokens) {
	SampleArgs a{};
	a.logits = s->logits;
	a.V = s->m->cfg.n_vocab;
	a.tok_out = s->tok;
	a.tok_log = log_tokens ? s->tok_log : nullptr;
	a.log_count = s->log_count;
	a.log_cap = s->log_cap;
	a.B = s->B;
	a.minp = minp;
	a.temp = temp;
	a.randf = s->randf;
	a.randf_count = s->randf_count;
	a.randf_cap = s->randf_cap;
	return a;
}

int enqueue_sampler(tg_state *s, float minp, float temp, bool log_tokens) {
	SampleArgs a = sample_args(s, minp, temp, log_tokens);
	if (minp < 1.0f && s->mega_ok && s->B == 1 && env_int("TG_MINP_GRID", 1)) {
		// one sequence: the row is spread over the whole GPU, sums ordered like the persistent kernel's sampler
		TG_CUDA(cudaMemsetAsync(s->mg_bar + 8, 0, 4, s->stream));
		unsigned *bar = s->mg_bar + 8;
		float *part = s->mg_samp_f;
		float *probs = s->mg_probs;
		int *err = s->err_flag;
		void *params[] = {&a, &bar, &part, &probs, &err};
		TG_CUDA(cudaLaunchCooperativeKernel((void *)minp_grid_kernel, dim3(s->mega_grid), dim3(SG_THREADS), params, 0, s->stream));
		count_launch();
		return check_launch("minp_grid");
	}
	if (minp < 1.0f) {  // transformer.hpp:208,229: min-p sampling iff minp < 1
		minp_kernel<<<s->B, SM_THREADS, 0, s->stream>>>(a);
		count_launch();
		return check_launch("minp");
	}
	launch_k(argmax_kernel, dim3(s->B), dim3(SM_THREADS), 0, s->stream, a);
	count_launch();
	return check_launch("argmax");
}

// the pinned staging buffer may be overwritten only when no enqueued copy still reads it
int staging_acquire(tg_state *s) {
	if (s->staging_busy) {
		TG_CUDA(cudaStreamSynchronize(s->stream));
		s->staging_busy = false;
	}
	return TG_OK;
}

// the error word a kernel left (read back by the caller) -> return code; clears the word on the device
int report_err_flag(tg_state *s, int flag) {
	if (flag) {
		cudaMemsetAsync(s->err_flag, 0, 4, s->stream);
		s->ps_clean = false;  // a launch that gave up leaves its hand-off words and barrier count anywhere
		if (flag > 0xFF) {  // the persistent kernel reports where it gave up above the code
			const int where = flag >> 8;
			const char *what = (flag & 0xFF) == 3 ? "bulk-copy" : ((flag & 0xFF) == 4 ? "grid-barrier" : "hand-off");
			return fail(TG_ECUDA, std::string("persistent kernel: a ") + what + " wait ran out (layer " + std::to_string(where >> 4) +
			                          ", phase " + std::to_string(where & 15) + ")");
		}
		if (flag == 1) return fail(TG_EINVAL, "token id out of range");
		if (flag == 2) return fail(TG_ESTATE, "global KV cache full (max_pos_global reached)");
		if (flag == 6) return fail(TG_ECUDA, "tensor-core GEMM: a pipeline wait ran out");
		if (flag == 5) return fail(TG_ECUDA, "persistent kernel: a hand-off flag wait ran out");
		return fail(TG_ECUDA, flag == 3 ? "persistent kernel: a TMA wait ran out" : "persistent kernel: a grid barrier wait ran out");
	}
	return TG_OK;
}

int check_err_flag(tg_state *s) {
	TG_CUDA(cudaMemcpyAsync(s->host_pin + 8192, s->err_flag, 4, cudaMemcpyDeviceToHost, s->stream));
	TG_CUDA(cudaStreamSynchronize(s->stream));
	s->staging_busy = false;
	return report_err_flag(s, s->host_pin[8192]);
}

int ensure_log(tg_state *s, int steps) {
	if (steps <= s->log_cap) return TG_OK;
	if (s->tok_log) cudaFree(s->tok_log);
	s->tok_log = nullptr;
	TG_CUDA(cudaMalloc(&s->tok_log, size_t(steps) * s->B * 4));
	s->log_cap = steps;
	return TG_OK;
}


// K-split of the tensor-core GEMM: enough CTAs to fill the GPU, accumulation chains of at most 24
// K-blocks (768 rows) for accuracy, as far as the partial-sum buffer allows.
constexpr size_t TC_TICKETS = 4096;
// ctas = CTAs of one split (column tiles x row-tile groups of the chosen tile shape)
int tc_pick_split(int ctas, int M, int K, int N, size_t partial_floats, int max_split) {
	const int k_blocks = K / TC_BK;
	// accumulation chains are kept to <= 24 K-blocks; a CTA keeps two accumulators per tile (first / second half of
	// its K range), so it can take up to 48 K-blocks
	// split only while every split still fits one wave (ctas * splits <= SMs): a second, partly filled wave
	// costs as much as the split saves
	const int fit = std::max(1, env_int("TG_GEMM_SPLIT_CEIL", 0) ? (g_num_sms + ctas - 1) / ctas : g_num_sms / ctas);
	const int need = (k_blocks + 47) / 48;
	// the largest divisor of the K-block count that still fits one wave; if the chain limit asks for more,
	// the smallest divisor that satisfies it
	int best = 1;
	for (int ns = 1; ns <= std::min(k_blocks, max_split); ns++) {
		if (k_blocks % ns) continue;
		if (ns > 1 && size_t(ns) * M * N > partial_floats) break;
		if (ns > fit && best >= need) break;
		best = ns;
	}
	return best;
}

size_t tc_pack_bytes(int M, int K) {
	const size_t m_tiles = (size_t(M) + TC_BM - 1) / TC_BM;
	return 3 * m_tiles * size_t(K / TC_BK) * TC_TILE_BYTES;
}

// packed operands of the tensor-core prefill attention for one prompt of S tokens: Q (4 S rows), K (S rows), V
struct AttnTcPlan {
	int q_tiles, k_tiles, v_blocks;
	size_t q_bytes, k_bytes, v_bytes;
	size_t total() const { return q_bytes + k_bytes + v_bytes; }
};
AttnTcPlan attn_tc_plan(int S) {
	AttnTcPlan p;
	p.q_tiles = (4 * S + TC_BM - 1) / TC_BM;
	p.k_tiles = (S + TC_BM - 1) / TC_BM;
	p.v_blocks = 4 * ((S + AT_TC_KT - 1) / AT_TC_KT);  // 16 keys each
	p.q_bytes = size_t(3) * p.q_tiles * 8 * TC_TILE_BYTES;
	p.k_bytes = size_t(3) * p.k_tiles * 8 * TC_TILE_BYTES;
	p.v_bytes = size_t(3) * p.v_blocks * AT_TC_VBYTES;
	return p;
}

int pack_activations(const float *A, int M, int K, const TcScratch &sc, cudaStream_t st) {
	if (tc_pack_bytes(M, K) > sc.apack_bytes) return fail(TG_ENOMEM, "tensor-core GEMM scratch too small");
	const int m_tiles = (M + TC_BM - 1) / TC_BM;
	const size_t chunks = size_t(m_tiles) * TC_BM * (K / 8);
	const unsigned grid = unsigned(std::min<size_t>((chunks + 255) / 256, size_t(g_num_sms) * 16));
	launch_k(split_pack_kernel, dim3(grid), dim3(256), 0, st, A, sc.apack, M, K, m_tiles);
	count_launch();
	return check_launch("split_pack");
}

// One launch for up to three weight matrices with the same K that multiply the same packed A
// (q|k|v, up|gate): more column tiles per launch, one split-K reduce instead of three.
// raw_nsplit != null: the kernel leaves raw partial sums in sc.partial ([nsplit][M][sum of N]) for a consumer
// kernel that adds the splits and scales itself; *raw_nsplit receives the split count, no reduce is launched.
int launch_gemm_tc_group(int ng, float *const *Cs, const QW *const *ws, const int *ldcs, int M, const TcScratch &sc,
                         cudaStream_t st, int max_split = 1 << 30, int *raw_nsplit = nullptr) {
	static bool configured[TG_MAX_DEVICES] = {false};
	const int dev = current_device_slot();
	if (!configured[dev]) {
		TG_CUDA(cudaFuncSetAttribute(qgemm_tc_kernel<2, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcShape<2, 128>::SMEM));
		TG_CUDA(cudaFuncSetAttribute(qgemm_tc_kernel<1, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcShape<1, 256>::SMEM));
		configured[dev] = true;
	}
	// tile shape: beyond one row tile the wide shape (one row tile x 256 columns) wins: a 256-column MMA
	// keeps the tensor pipe busier than two of 128 and every fetched A tile is used twice as often
	const int m_tiles_all = (M + TC_BM - 1) / TC_BM;
	const bool wide = M >= env_int("TG_GEMM_WIDE_MIN_M", 129);
	const int bn = wide ? 256 : 128, mt_cta = wide ? 1 : 2;
	CUtensorMap wmap[3];
	GemmTcArgs a{};
	ReduceGroups rg{};
	int ntot = 0, tiles = 0;
	const int K = ws[0]->K;
	for (int g = 0; g < 3; g++) {
		const int gg = std::min(g, ng - 1);  // unused slots repeat the last matrix (never selected)
		if (ws[gg]->K != K) return fail(TG_ESHAPE, "grouped GEMM: the matrices must share K");
		TG_TRY(make_tmap(&wmap[g], ws[gg]->q, K, ws[gg]->N, bn, TC_BK, ws[gg]->ld));
		if (g < ng) {
			a.col0[g] = ntot;
			a.ncols[g] = ws[g]->N;
			a.scales[g] = ws[g]->s;
			a.C[g] = Cs[g];
			a.ldc[g] = (ldcs && ldcs[g] > 0) ? ldcs[g] : ws[g]->N;
			ntot += ws[g]->N;
			tiles += (ws[g]->N + bn - 1) / bn;
			a.tile_end[g] = tiles;
			rg.col0[g] = a.col0[g];
			rg.scales[g] = a.scales[g];
			rg.C[g] = a.C[g];
			rg.ldc[g] = a.ldc[g];
		} else {
			a.col0[g] = ntot;
			a.tile_end[g] = INT_MAX;
			a.ncols[g] = 0;
			a.scales[g] = a.scales[ng - 1];
			a.C[g] = a.C[ng - 1];
			a.ldc[g] = a.ldc[ng - 1];
		}
	}
	rg.ngroups = ng;
	rg.col0[ng] = ntot;
	for (int g = ng + 1; g < 4; g++) rg.col0[g] = INT_MAX;
	a.ngroups = ng;
	a.apack = sc.apack;
	a.M = M;
	a.N = ntot;
	a.K = K;
	a.m_tiles = m_tiles_all;
	a.nsplit = tc_pick_split(tiles * ((m_tiles_all + mt_cta - 1) / mt_cta), M, K, ntot, sc.partial_floats, std::min(max_split, env_int("TG_GEMM_MAX_SPLIT", sc.max_split)));
	a.partial = sc.partial;
	a.err = sc.err;
	a.top1 = sc.top1;
	a.top1_col0 = sc.top1_col0;
	if (a.top1 && (a.nsplit != 1 || raw_nsplit)) return fail(TG_EINVAL, "top-1 epilogue needs an unsplit K");
	dim3 grid(tiles, (a.m_tiles + mt_cta - 1) / mt_cta, a.nsplit);
	const bool fused = !raw_nsplit && sc.tickets && a.nsplit > 1 && a.nsplit <= sc.fused_max_split && size_t(grid.x) * grid.y <= TC_TICKETS;
	a.tickets = fused ? sc.tickets : nullptr;
	a.raw = raw_nsplit ? 1 : 0;
	a.halves = env_int("TG_GEMM_HALVES", 2);
	if (raw_nsplit) {
		if (size_t(a.nsplit) * M * ntot > sc.partial_floats) return fail(TG_ENOMEM, "tensor-core GEMM partial-sum scratch too small");
		*raw_nsplit = a.nsplit;
	}
	if (wide)
		launch_k(qgemm_tc_kernel<1, 256>, grid, dim3(TC_THREADS), TcShape<1, 256>::SMEM, st, wmap[0], wmap[1], wmap[2], a);
	else
		launch_k(qgemm_tc_kernel<2, 128>, grid, dim3(TC_THREADS), TcShape<2, 128>::SMEM, st, wmap[0], wmap[1], wmap[2], a);
	count_launch();
	TG_TRY(check_launch("qgemm_tc"));
	if (a.nsplit > 1 && !fused && !raw_nsplit) {
		const size_t n = size_t(M) * ntot;
		qgemm_splitk_reduce_groups_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(rg, sc.partial, M, ntot, a.nsplit);
		count_launch();
		TG_TRY(check_launch("qgemm_reduce"));
	}
	return TG_OK;
}
int launch_gemm_tc(float *C, const QW &w, int M, const TcScratch &sc, cudaStream_t st, int ldc = 0, int max_split = 1 << 30) {
	float *Cs[1] = {C};
	const QW *ws[1] = {&w};
	const int ldcs[1] = {ldc};
	return launch_gemm_tc_group(1, Cs, ws, ldcs, M, sc, st, max_split);
}

// ------------------------------------------------------------- batched decode step
// For larger batches the per-token work is the prefill's: every weight matrix is read once per
// step for all sequences by the tensor-core GEMM (M = batch), the norms run row-wise, and only
// the attention is per sequence (each against its own cache, positions read on the device).
int batched_setup(tg_state *s) {
	const tg_config &c = s->m->cfg;
	const int B = s->B, D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab, qd = c.n_head * c.head_dim;
	TG_CUDA(cudaMalloc(&s->bx, size_t(B) * D * 4));
	TG_CUDA(cudaMalloc(&s->bup, size_t(B) * I * 4));
	s->btc.apack_bytes = tc_pack_bytes(B, std::max(I, std::max(D, qd)));
	TG_CUDA(cudaMalloc(&s->btc.apack, s->btc.apack_bytes));
	s->btc.partial_floats = std::min(size_t(24) * B * std::max(I, qd), size_t(1) << 28);
	TG_CUDA(cudaMalloc(&s->btc.partial, s->btc.partial_floats * 4));
	TG_CUDA(cudaMalloc(&s->btc.tickets, TC_TICKETS * sizeof(unsigned)));
	TG_CUDA(cudaMemset(s->btc.tickets, 0, TC_TICKETS * sizeof(unsigned)));
	s->btc.max_split = env_int("TG_BATCH_MAX_SPLIT", 9);
	s->btc.err = s->err_flag;
	(void)V;
	s->batched_ok = true;
	return TG_OK;
}

int enqueue_decode_batched(tg_state *s, bool with_lm_head) {
	struct PdlOff {
		bool was = g_pdl_scope_off;
		PdlOff() { g_pdl_scope_off = true; }
		~PdlOff() { g_pdl_scope_off = was; }
	} pdl_off;
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int B = s->B, D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim;
	cudaStream_t st = s->stream;
	const GeluLut lut = make_lut(m);
	float *h = s->h[0];
	EmbedArgs ea;
	ea.wte = m->wte;
	ea.scales = m->wte_s;
	ea.tok = s->tok;
	ea.h = h;
	ea.step_pos = s->step_pos;
	ea.next_pos = s->next_pos;
	ea.err_flag = s->err_flag;
	ea.D = D;
	ea.V = V;
	ea.sqrtD = float(std::sqrt(double(D)));
	launch_k(embed_decode_kernel, dim3(B), dim3(256), 0, st, ea);
	count_launch();
	const int m_tiles = (B + TC_BM - 1) / TC_BM;
	// t: finished matrix (nsplit 0) or the raw partial sums of the GEMM before (nsplit >= 1, column scales tscale)
	auto resnorm_pack = [&](const float *t, const float *w_post, const float *w_pre, int nsplit, const float *tscale) {
		launch_k(resnorm_pack_kernel<256>, dim3(m_tiles * TC_BM), dim3(256), 0, st, h, t, w_post, w_pre, s->btc.apack, B, D, m_tiles, nsplit, D, tscale);
		count_launch();
	};
	auto gemm_raw = [&](int ng, const QW *const *ws, int *ns) -> int {
		float *Cs[3] = {nullptr, nullptr, nullptr};
		return launch_gemm_tc_group(ng, Cs, ws, nullptr, B, s->btc, st, 1 << 30, ns);
	};
	resnorm_pack(nullptr, nullptr, m->layers[0].attn_pre, 0, nullptr);
	for (int l = 0; l < c.n_layers; l++) {
		const LayerW &w = m->layers[l];
		int ns_qkv = 0;
		{
			const QW *ws[3] = {&w.Q, &w.K, &w.V};
			TG_TRY(gemm_raw(3, ws, &ns_qkv));  // raw partial sums: the attention kernel adds the splits and scales
		}
		{
			AttnArgs a{};
			a.qkv = s->btc.partial;
			a.qkv_nsplit = ns_qkv;
			a.qkv_B = B;
			a.sq = w.Q.s;
			a.sk = w.K.s;
			a.sv = w.V.s;
			a.rmsq = w.rmsq;
			a.rmsk = w.rmsk;
			a.cosT = m->rope[w.is_local ? 1 : 0][0];
			a.sinT = m->rope[w.is_local ? 1 : 0][1];
			a.slots = s->slots[l];
			a.kcache = s->kcache[l];
			a.vcache = s->vcache[l];
			a.is_local = w.is_local ? 1 : 0;
			a.step_pos = s->step_pos;
			a.ring_base = s->ring_base;
			a.nsplit = w.is_local ? s->attn_nsplit_local : s->attn_nsplit_global;
			a.part = s->attn_part;
			a.tickets = s->attn_tickets;
			a.out = s->attn_out;
			a.err_flag = s->err_flag;
			launch_k(attn_decode_kernel, dim3(a.nsplit, B), dim3(AT_THREADS), 0, st, a);
			count_launch();
			TG_TRY(check_launch("attn_decode"));
		}
		TG_TRY(pack_activations(s->attn_out, B, qd, s->btc, st));
		int ns = 0;
		{
			const QW *ws[1] = {&w.O};
			TG_TRY(gemm_raw(1, ws, &ns));
		}
		resnorm_pack(s->btc.partial, w.attn_post, w.mlp_pre, ns, w.O.s);
		{
			const QW *ws[2] = {&w.U, &w.G};
			TG_TRY(gemm_raw(2, ws, &ns));
		}
		launch_k(geglu_pack_kernel, dim3(unsigned((size_t(m_tiles) * TC_BM * (I / 8) + 255) / 256)), dim3(256), 0, st, (const float *)nullptr, (const float *)s->btc.partial, s->btc.apack, B, I, m_tiles, lut, ns, w.U.s, w.G.s);
		count_launch();
		{
			const QW *ws[1] = {&w.Dn};
			TG_TRY(gemm_raw(1, ws, &ns));
		}
		resnorm_pack(s->btc.partial, w.mlp_post, l + 1 < c.n_layers ? m->layers[l + 1].attn_pre : nullptr, ns, w.Dn.s);
		TG_TRY(check_launch("batched layer"));
	}
	launch_k(rmsnorm_rows_kernel, dim3(B), dim3(256), 0, st, s->xnorm, (const float *)h, m->final_norm, (const float *)nullptr, D);
	count_launch();
	if (with_lm_head) {
		TG_TRY(pack_activations(s->xnorm, B, D, s->btc, st));
		TG_TRY(launch_gemm_tc(s->logits, m->lm_head, B, s->btc, st, 0, 1));
	}
	return check_launch("batched decode");
}

int launch_gemm(float *C, const float *A, const QW &w, int M, float *partial, size_t partial_floats, cudaStream_t st) {
	const int K = w.K, N = w.N;
	dim3 grid(N / GM_BN, (M + GM_BM - 1) / GM_BM, 1);
	int ctas = grid.x * grid.y;
	int nsplit = 1;
	const int units = K / GM_BK;
	if (ctas < g_num_sms) {
		int want = (2 * g_num_sms + ctas - 1) / ctas;
		for (int ns = 1; ns <= units; ns++)
			if (units % ns == 0 && size_t(ns) * M * N <= partial_floats) {
				nsplit = ns;
				if (ns >= want) break;
			}
	}
	grid.z = nsplit;
	qgemm_simt_kernel<<<grid, 256, 0, st>>>(C, A, w.q, w.s, M, K, N, K / nsplit, partial);
	count_launch();
	TG_TRY(check_launch("qgemm_simt"));
	if (nsplit > 1) {
		size_t n = size_t(M) * N;
		qgemm_splitk_reduce_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(C, partial, w.s, M, N, nsplit, N);
		count_launch();
		TG_TRY(check_launch("qgemm_reduce"));
	}
	return TG_OK;
}

// prefill of the nb sequences b .. b + nb - 1, S tokens each, already in s->pf_ids (device). Their rows are
// stacked (row = sequence * S + position): embedding, norms, GEMMs and GeGLU work on all nb * S rows at once —
// a GEMM over 178 rows runs at a sixth of the tensor throughput of one over thousands — and only the
// per-sequence steps (RoPE positions, cache fill, causal attention) index by sequence (blockIdx.y).
int enqueue_prefill_seq(tg_state *s, int b, int S_seq, int nb = 1) {
	const int S = S_seq * nb;  // rows
	tg_model *m = s->m;
	const tg_config &c = m->cfg;
	const int D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	cudaStream_t st = s->stream;
	const GeluLut lut = make_lut(m);
	// scratch carve-up
	float *p = s->pf;
	float *h = p;        p += size_t(S) * D;
	float *xn = p;       p += size_t(S) * D;
	float *q = p;        p += size_t(S) * qd;
	float *k = p;        p += size_t(S) * kd;
	float *v = p;        p += size_t(S) * kd;
	float *ao = p;       p += size_t(S) * qd;
	float *tt = p;       p += size_t(S) * D;
	float *up = p;       p += size_t(S) * I;
	float *gate = p;     p += size_t(S) * I;
	const bool use_tc = env_int("TG_GEMM_TC", 1) != 0;
	TcScratch tc;
	if (use_tc) {
		tc.apack = reinterpret_cast<__nv_bfloat16 *>(p);
		tc.apack_bytes = tc_pack_bytes(S, std::max(I, std::max(D, qd)));
		tc.err = s->err_flag;
		p += (tc.apack_bytes + 3) / 4;
	}
	// long prompts: attention on the tensor cores, from packed copies of q, k and v, one sequence after the other
	// (from 640 tokens on: below, the three packing launches cost what the tensor cores save)
	const bool attn_tc = use_tc && S_seq > env_int("TG_ATTN_SMALL_MAX", 384) && env_int("TG_ATTN_TC", 1) &&
	                     S_seq >= env_int("TG_ATTN_TC_MIN", 640);
	const AttnTcPlan atp = attn_tc_plan(S_seq);
	__nv_bfloat16 *at_q = nullptr, *at_k = nullptr, *at_v = nullptr;
	if (attn_tc) {
		p = reinterpret_cast<float *>((uintptr_t(p) + 1023) & ~uintptr_t(1023));
		at_q = reinterpret_cast<__nv_bfloat16 *>(p);
		at_k = reinterpret_cast<__nv_bfloat16 *>(reinterpret_cast<uint8_t *>(p) + atp.q_bytes);
		at_v = reinterpret_cast<__nv_bfloat16 *>(reinterpret_cast<uint8_t *>(p) + atp.q_bytes + atp.k_bytes);
		p += (atp.total() + 3) / 4;
	}
	float *part = p;
	size_t part_floats = s->pf_floats - size_t(part - s->pf);
	tc.partial = part;
	tc.partial_floats = part_floats;
	// C = A . W for one weight; `fresh` = A differs from the previous call and must be packed again
	auto gemm = [&](float *C, const float *A, const QW &w, bool fresh) -> int {
		if (!use_tc) return launch_gemm(C, A, w, S, part, part_floats, st);
		if (fresh) TG_TRY(pack_activations(A, S, w.K, tc, st));
		return launch_gemm_tc(C, w, S, tc, st);
	};

	launch_k(embed_prefill_kernel, dim3(S), dim3(256), 0, st, m->wte, m->wte_s, (const int *)(s->pf_ids + size_t(b) * S_seq), h, S, D, V,
	         float(std::sqrt(double(D))), s->err_flag);
	count_launch();
	TG_TRY(check_launch("embed_prefill"));
	const int m_tiles = (S + TC_BM - 1) / TC_BM;
	// Tensor-core path: the norms are fused with the operand packing of the GEMM that follows them
	// (resnorm_pack_kernel, geglu_pack_kernel), so a layer is 7 GEMMs (+ their split-K reduces) and 6 other launches.
	auto resnorm_pack = [&](const float *t, const float *w_post, const float *w_pre, int nsplit, const float *tscale) {
		if (S >= env_int("TG_RESNORM_NARROW_MIN", 1024))
			launch_k(resnorm_pack_kernel<128>, dim3(m_tiles * TC_BM), dim3(128), 0, st, h, t, w_post, w_pre, tc.apack, S, D, m_tiles, nsplit, D, tscale);
		else
			launch_k(resnorm_pack_kernel<256>, dim3(m_tiles * TC_BM), dim3(256), 0, st, h, t, w_post, w_pre, tc.apack, S, D, m_tiles, nsplit, D, tscale);
		count_launch();
	};
	auto gemm_raw = [&](int ng, const QW *const *ws, int *ns) -> int {
		float *Cs[3] = {nullptr, nullptr, nullptr};
		return launch_gemm_tc_group(ng, Cs, ws, nullptr, S, tc, st, 1 << 30, ns);
	};
	if (use_tc) {
		if (tc_pack_bytes(S, std::max(I, std::max(D, qd))) > tc.apack_bytes) return fail(TG_ENOMEM, "tensor-core GEMM scratch too small");
		resnorm_pack(nullptr, nullptr, m->layers[0].attn_pre, 0, nullptr);
	}
	for (int l = 0; l < c.n_layers; l++) {
		const LayerW &w = m->layers[l];
		const int slots = s->slots[l];
		int ns_qkv = 0;  // > 0: q|k|v are raw partial sums, finished by the norm + RoPE kernel
		if (use_tc) {
			const QW *ws[3] = {&w.Q, &w.K, &w.V};
			TG_TRY(gemm_raw(3, ws, &ns_qkv));
		} else {
			rmsnorm_rows_kernel<<<S, 256, 0, st>>>(xn, h, w.attn_pre, nullptr, D);
			count_launch();
			TG_TRY(gemm(q, xn, w.Q, true));
			TG_TRY(gemm(k, xn, w.K, false));
			TG_TRY(gemm(v, xn, w.V, false));
		}
		launch_k(qk_norm_rope_prefill_kernel, dim3(S_seq, nb), dim3(192), 0, st, q, k, v, w.rmsq, w.rmsk, m->rope[w.is_local ? 1 : 0][0],
		         m->rope[w.is_local ? 1 : 0][1], s->kcache[l] + size_t(b) * slots * AT_HD, s->vcache[l] + size_t(b) * slots * AT_HD, S_seq,
		         slots, (const float *)tc.partial, ns_qkv, w.Q.s, w.K.s, w.V.s, S, size_t(slots) * AT_HD);
		count_launch();
		if (S_seq <= env_int("TG_ATTN_SMALL_MAX", 384))  // short prompts: a (query, head)'s keys split over four warps, S/2 CTAs
			launch_k(attn_prefill_small_kernel, dim3((S_seq + 1) / 2, nb), dim3(APS_THREADS), 0, st, ao, q, k, v, S_seq, w.is_local ? 1 : 0, c.n_pos_local);
		else if (attn_tc) {
			static bool at_configured[TG_MAX_DEVICES] = {false};
			const int dev = current_device_slot();
			if (!at_configured[dev]) {
				TG_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_TC_SMEM));
				at_configured[dev] = true;
			}
			auto pack_rows = [&](const float *src, __nv_bfloat16 *dst, int rows, int tiles) {
				const size_t chunks = size_t(tiles) * TC_BM * (256 / 8);
				launch_k(split_pack_kernel, dim3(unsigned(std::min<size_t>((chunks + 255) / 256, size_t(g_num_sms) * 16))), dim3(256), 0, st, src, dst, rows,
				         256, tiles);
				count_launch();
			};
			for (int i = 0; i < nb; i++) {  // (the packed copies are reused from sequence to sequence: stream order)
			const float *qi = q + size_t(i) * S_seq * qd, *ki = k + size_t(i) * S_seq * kd, *vi = v + size_t(i) * S_seq * kd;
			pack_rows(qi, at_q, 4 * S_seq, atp.q_tiles);  // rows = (query, head) pairs as they lie in q [S][4][256]
			pack_rows(ki, at_k, S_seq, atp.k_tiles);
			launch_k(attn_pack_v_kernel, dim3(unsigned(std::min<size_t>((size_t(atp.v_blocks) * 512 + 255) / 256, size_t(g_num_sms) * 16))), dim3(256), 0,
			         st, vi, at_v, S_seq, atp.v_blocks);
			count_launch();
			AttnTcArgs aa{};
			aa.qp = at_q;
			aa.kp = at_k;
			aa.vp = at_v;
			aa.o = ao + size_t(i) * S_seq * qd;
			aa.S = S_seq;
			aa.q_tiles = atp.q_tiles;
			aa.k_tiles = atp.k_tiles;
			aa.v_blocks = atp.v_blocks;
			aa.is_local = w.is_local ? 1 : 0;
			aa.window = c.n_pos_local;
			aa.err = s->err_flag;
			launch_k(attn_prefill_tc_kernel, dim3(atp.q_tiles), dim3(AT_TC_THREADS), size_t(AT_TC_SMEM), st, aa);
			if (i + 1 < nb) count_launch();
			}
		} else
			if (env_int("TG_ATTN_BLOCK4", 1)) {  // long prompts: four keys per step (TG_ATTN_BLOCK4=0: the per-key kernel)
				static bool configured[TG_MAX_DEVICES] = {false};
				const int dev = current_device_slot();
				if (!configured[dev]) {
					TG_CUDA(cudaFuncSetAttribute(attn_prefill_blk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_BLK_SMEM));
					configured[dev] = true;
				}
				launch_k(attn_prefill_blk_kernel, dim3((S_seq + 7) / 8, nb), dim3(256), AP_BLK_SMEM, st, ao, q, k, v, S_seq, w.is_local ? 1 : 0, c.n_pos_local);
			} else
				attn_prefill_kernel<<<dim3((S_seq + 7) / 8, nb), 256, 0, st>>>(ao, q, k, v, S_seq, w.is_local ? 1 : 0, c.n_pos_local);
		count_launch();
		TG_TRY(check_launch("attn_prefill"));
		if (use_tc) {
			// the O, up|gate and down GEMMs leave raw K-split partial sums; the kernel that consumes them adds the splits
			int ns = 0;
			TG_TRY(pack_activations(ao, S, qd, tc, st));
			{
				const QW *ws[1] = {&w.O};
				TG_TRY(gemm_raw(1, ws, &ns));
			}
			resnorm_pack(tc.partial, w.attn_post, w.mlp_pre, ns, w.O.s);
			{
				const QW *ws[2] = {&w.U, &w.G};
				TG_TRY(gemm_raw(2, ws, &ns));
			}
			launch_k(geglu_pack_kernel, dim3(unsigned(std::min<size_t>((size_t(m_tiles) * TC_BM * (I / 8) + 255) / 256, 65535 * 16))), dim3(256), 0, st,
			         (const float *)nullptr, (const float *)tc.partial, tc.apack, S, I, m_tiles, lut, ns, w.U.s, w.G.s);
			count_launch();
			{
				const QW *ws[1] = {&w.Dn};
				TG_TRY(gemm_raw(1, ws, &ns));
			}
			resnorm_pack(tc.partial, w.mlp_post, l + 1 < c.n_layers ? m->layers[l + 1].attn_pre : nullptr, ns, w.Dn.s);
		} else {
			TG_TRY(gemm(tt, ao, w.O, true));
			rmsnorm_rows_kernel<<<S, 256, 0, st>>>(h, tt, w.attn_post, h, D);
			count_launch();
			rmsnorm_rows_kernel<<<S, 256, 0, st>>>(xn, h, w.mlp_pre, nullptr, D);
			count_launch();
			TG_TRY(gemm(up, xn, w.U, true));
			TG_TRY(gemm(gate, xn, w.G, false));
			size_t n = size_t(S) * I;
			geglu_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(gate, up, n, lut);
			count_launch();
			TG_TRY(gemm(tt, gate, w.Dn, true));
			rmsnorm_rows_kernel<<<S, 256, 0, st>>>(h, tt, w.mlp_post, h, D);
			count_launch();
		}
		TG_TRY(check_launch("prefill layer"));
	}
	// lm_head on the last position of every sequence (modules.hpp:232-240)
	if (nb >= 4 && use_tc) {
		// a group: the last rows are gathered (one strided copy), normed, and scored by ONE GEMM over the
		// vocabulary matrix, as the batched decode step does — not nb matvecs that each stream its 302 MB
		float *last = xn;  // [nb][D] (xn is free: the tensor-core path packs its norm outputs directly)
		TG_CUDA(cudaMemcpy2DAsync(last, size_t(D) * 4, h + size_t(S_seq - 1) * D, size_t(S_seq) * D * 4, size_t(D) * 4, nb, cudaMemcpyDeviceToDevice, st));
		launch_k(rmsnorm_rows_kernel, dim3(nb), dim3(256), 0, st, s->xnorm + size_t(b) * D, (const float *)last, m->final_norm, (const float *)nullptr, D);
		count_launch();
		TG_TRY(pack_activations(s->xnorm + size_t(b) * D, nb, D, tc, st));
		TG_TRY(launch_gemm_tc(s->logits + size_t(b) * V, m->lm_head, nb, tc, st, 0, 1));
		return TG_OK;
	}
	for (int i = 0; i < nb; i++) {
		MvArgs a{};
		a.seg[0] = MvSeg{m->lm_head.q, m->lm_head.s, V, 0, 0};
		a.nseg = 1;
		a.ntiles = V / MV_TN;
		a.K = D;
		a.kc = s->plan_lm.kc;
		a.nsplit = s->plan_lm.nsplit;
		a.B = 1;
		a.part_stride = V;
		a.out_stride = V;
		a.h = h + (size_t(i + 1) * S_seq - 1) * D;
		a.w_pre = m->final_norm;
		a.x_out = s->xnorm + size_t(b + i) * D;
		a.partial = s->partial;
		a.tickets = s->tickets;
		a.out = s->logits + size_t(b + i) * V;
		TG_TRY(launch_mv(a, PRO_NORM, EPI_SCALE, st));
	}
	return TG_OK;
}

}  // namespace

// ===================================================================== C ABI
extern "C" {

const char *tg_last_error(void) { return g_err.c_str(); }
const char *tg_version(void) { return "tiny-gemma_b200 0.1 (sm_100a)"; }

int tg_device_count(int *count) {
	if (!count) return fail(TG_EINVAL, "count is null");
	int n = 0;
	cudaError_t e = cudaGetDeviceCount(&n);
	if (e != cudaSuccess) {
		cudaGetLastError();
		n = 0;
	}
	*count = n;
	return TG_OK;
}

int tg_config_by_name(const char *name, tg_config *out) {
	if (!name || !out) return fail(TG_EINVAL, "null argument");
	// reference config.hpp:46-48
	if (std::strcmp(name, "270m") == 0) {
		*out = tg_config{640, 2048, 18, 262144, 32768, 512, 256, 4, 1, 1000000.0f, 10000.0f, 6};
		return TG_OK;
	}
	if (std::strcmp(name, "1B") == 0) {
		*out = tg_config{1152, 6912, 26, 262144, 32768, 512, 256, 4, 1, 1000000.0f, 10000.0f, 6};
		return TG_OK;
	}
	return fail(TG_EINVAL, std::string("unknown model size: ") + name);
}

int tg_model_file_bytes(const tg_config *cfg, size_t *nbytes) {
	if (!cfg || !nbytes) return fail(TG_EINVAL, "null argument");
	*nbytes = model_file_bytes(*cfg);
	return TG_OK;
}

int tg_model_create(const tg_config *cfg, int device, tg_model **out) {
	if (!cfg || !out) return fail(TG_EINVAL, "null argument");
	const tg_config &c = *cfg;
	if (c.head_dim != 256 || c.n_head != 4 || c.n_kv != 1)
		return fail(TG_ESHAPE, "kernels are specialised for 4 query heads, 1 KV head, head_dim 256");
	if (!supported_k(c.hidden_size) || !supported_n(c.hidden_size) || !supported_k(c.intermediate_size) ||
	    !supported_n(c.intermediate_size) || c.n_vocab % 8192 != 0 || c.n_layers < 1 || c.window_pattern < 1)
		return fail(TG_ESHAPE, "unsupported model dimensions");
	TG_TRY(ensure_device(device));
	tg_model *m = new tg_model();
	m->cfg = c;
	m->device = device;
	m->nbytes = model_file_bytes(c);
	cudaError_t e = cudaMalloc(&m->blob, m->nbytes);
	if (e != cudaSuccess) {
		delete m;
		return fail(TG_ENOMEM, std::string("cudaMalloc(weights): ") + cudaGetErrorString(e));
	}
	cudaMemset(m->blob, 0, m->nbytes);
	bind_model(m);
	*out = m;
	return TG_OK;
}

int tg_model_free(tg_model *m) {
	if (!m) return TG_OK;
	cudaSetDevice(m->device);
	cudaFree(m->blob);
	cudaFree(m->dec_tiled);
	cudaFree(m->ps_tiled);
	cudaFree(m->ps_lm);
	for (int i = 0; i < 2; i++)
		for (int j = 0; j < 2; j++) cudaFree(m->rope[i][j]);
	cudaFree(m->gelu);
	delete m;
	return TG_OK;
}

int tg_model_load_memory(tg_model *m, const void *bytes, size_t nbytes) {
	if (!m || !bytes) return fail(TG_EINVAL, "null argument");
	if (nbytes < m->nbytes) return fail(TG_EIO, "weights image shorter than the model needs");
	TG_CUDA(cudaSetDevice(m->device));
	TG_CUDA(cudaMemcpy(m->blob, bytes, m->nbytes, cudaMemcpyHostToDevice));
	m->loaded = true;
	m->weights_version++;
	return TG_OK;
}

int tg_model_load_file(tg_model *m, const char *path) {
	if (!m || !path) return fail(TG_EINVAL, "null argument");
	FILE *f = std::fopen(path, "rb");
	if (!f) return fail(TG_EIO, "Could not open file.");
	TG_CUDA(cudaSetDevice(m->device));
	// stream the file through two pinned buffers so the disk read and the copy overlap
	const size_t CH = size_t(64) << 20;
	uint8_t *pin[2] = {nullptr, nullptr};
	cudaStream_t st;
	cudaEvent_t ev[2];
	if (cudaMallocHost(&pin[0], CH) != cudaSuccess || cudaMallocHost(&pin[1], CH) != cudaSuccess) {
		std::fclose(f);
		cudaFreeHost(pin[0]);
		return fail(TG_ENOMEM, "cudaMallocHost(staging)");
	}
	cudaStreamCreate(&st);
	cudaEventCreate(&ev[0]);
	cudaEventCreate(&ev[1]);
	size_t off = 0;
	int rc = TG_OK;
	for (int i = 0; off < m->nbytes; i ^= 1) {
		size_t want = std::min(CH, m->nbytes - off);
		cudaEventSynchronize(ev[i]);
		size_t got = std::fread(pin[i], 1, want, f);
		if (got != want) {
			rc = fail(TG_EIO, "weights file is shorter than the model needs");
			break;
		}
		if (cudaMemcpyAsync(m->blob + off, pin[i], want, cudaMemcpyHostToDevice, st) != cudaSuccess) {
			rc = fail(TG_ECUDA, "cudaMemcpyAsync(weights)");
			break;
		}
		cudaEventRecord(ev[i], st);
		off += want;
	}
	cudaStreamSynchronize(st);
	std::fclose(f);
	cudaEventDestroy(ev[0]);
	cudaEventDestroy(ev[1]);
	cudaStreamDestroy(st);
	cudaFreeHost(pin[0]);
	cudaFreeHost(pin[1]);
	if (rc == TG_OK) {
		m->loaded = true;
		m->weights_version++;
	}
	return rc;
}

int tg_model_set_rope(tg_model *m, int is_local, const float *cos_host, const float *sin_host, int n_pos) {
	if (!m || !cos_host || !sin_host || n_pos <= 0) return fail(TG_EINVAL, "bad argument");
	// the kernels read row `position` for every position a state may reach (max_pos_global <= n_pos); the
	// reference's decode::RoPE always builds cfg.n_pos rows (decode.hpp:118-200), so a shorter table is refused
	if (n_pos < m->cfg.n_pos) return fail(TG_EINVAL, "RoPE table shorter than the model's n_pos");
	TG_CUDA(cudaSetDevice(m->device));
	const int i = is_local ? 1 : 0;
	size_t n = size_t(n_pos) * m->cfg.head_dim * 4;
	const float *src[2] = {cos_host, sin_host};
	for (int j = 0; j < 2; j++) {
		if (m->rope[i][j]) cudaFree(m->rope[i][j]);
		m->rope[i][j] = nullptr;
		TG_CUDA(cudaMalloc(&m->rope[i][j], n));
		TG_CUDA(cudaMemcpy(m->rope[i][j], src[j], n, cudaMemcpyHostToDevice));
	}
	m->rope_npos[i] = n_pos;
	return TG_OK;
}

int tg_model_set_gelu_table(tg_model *m, float mn, float mx, const float *table, int size) {
	if (!m || !table || size <= 0) return fail(TG_EINVAL, "bad argument");
	TG_CUDA(cudaSetDevice(m->device));
	if (m->gelu) cudaFree(m->gelu);
	m->gelu = nullptr;
	TG_CUDA(cudaMalloc(&m->gelu, size_t(size) * 4));
	TG_CUDA(cudaMemcpy(m->gelu, table, size_t(size) * 4, cudaMemcpyHostToDevice));
	m->gelu_min = mn;
	m->gelu_max = mx;
	m->gelu_size = size;
	m->gelu_eps = float(mx - mn) / float(size);  // ops.hpp:33
	return TG_OK;
}

int tg_model_build_tables(tg_model *m, int gelu_size) {
	if (!m || gelu_size <= 0) return fail(TG_EINVAL, "bad argument");
	const tg_config &c = m->cfg;
	const int hd = c.head_dim, half = hd / 2;
	std::vector<float> ct(size_t(c.n_pos) * hd), st(size_t(c.n_pos) * hd), freqs(half);
	for (int loc = 0; loc < 2; loc++) {
		// decode.hpp:176-201
		const float theta = loc ? c.rope_theta_local : c.rope_theta;
		for (int i = 0; i < half; i++) {
			float denom = std::pow(theta, float(2 * i) / hd);
			freqs[i] = float(1.0 / denom);
		}
		for (int p = 0; p < c.n_pos; p++)
			for (int d = 0; d < half; d++) {
				float outer = p * freqs[d];
				float cv = std::cos(outer), sv = std::sin(outer);
				ct[size_t(p) * hd + d] = cv;
				ct[size_t(p) * hd + d + half] = cv;
				st[size_t(p) * hd + d] = sv;
				st[size_t(p) * hd + d + half] = sv;
			}
		TG_TRY(tg_model_set_rope(m, loc, ct.data(), st.data(), c.n_pos));
	}
	// ops.hpp:16-39
	std::vector<float> tab(gelu_size);
	const float mn = -4.0f, mx = 4.0f, eps = float(mx - mn) / float(gelu_size);
	for (int i = 0; i < gelu_size; i++) {
		float a = mn + i * eps;
		double inner = double(0.7978845608f) * (double(a) + double(0.044715f) * std::pow(double(a), 3.0));
		tab[i] = float((0.5 * double(a)) * (1.0 + std::tanh(inner)));
	}
	return tg_model_set_gelu_table(m, mn, mx, tab.data(), gelu_size);
}

// ---------------------------------------------------------------- state
int tg_state_create(tg_model *m, int batch, int max_pos_global, tg_state **out) {
	if (!m || !out || batch < 1 || batch > 2048) return fail(TG_EINVAL, "bad argument (batch must be 1..2048)");
	if (max_pos_global <= 0) max_pos_global = m->cfg.n_pos;
	if (max_pos_global > m->cfg.n_pos) return fail(TG_EINVAL, "max_pos_global exceeds n_pos");
	TG_CUDA(cudaSetDevice(m->device));
	tg_state *s = new tg_state();
	s->m = m;
	s->B = batch;
	s->max_pos_global = max_pos_global;
	int rc = state_alloc(s);
	if (rc == TG_OK && batch >= env_int("TG_BATCH_TC_MIN", 4)) rc = batched_setup(s);
	if (rc == TG_OK && batch == 1 && env_int("TG_MEGA", 1)) {
		int mrc = mega_setup(s);
		if (mrc != TG_OK) {
			if (env_int("TG_MEGA", 1) == 2) rc = mrc;  // 2 = required
			s->mega_ok = false;
		} else if (env_int("TG_PERSIST", 1)) {
			// the dp4a kernel (kernels_persist.cuh) is the batch-1 decode path; a shape it has no plan for falls back
			// to the fp32-FMA kernel (kernels_mega.cuh), which TG_PERSIST=0 also selects
			int prc = persist_setup(s);
			if (prc != TG_OK) {
				if (env_int("TG_PERSIST", 1) == 2) rc = prc;  // 2 = required
				s->ps_ok = false;
			}
		}
	}
	if (rc != TG_OK) {
		std::string keep = g_err;
		tg_state_free(s);
		g_err = keep;
		return rc;
	}
	*out = s;
	return TG_OK;
}

int tg_state_free(tg_state *s) {
	if (!s) return TG_OK;
	cudaSetDevice(s->m->device);
	if (s->stream) cudaStreamSynchronize(s->stream);
	if (s->graph) cudaGraphExecDestroy(s->graph);
	for (float *p : s->kcache) cudaFree(p);
	for (float *p : s->vcache) cudaFree(p);
	cudaFree(s->h[0]);
	cudaFree(s->h[1]);
	cudaFree(s->qkv);
	cudaFree(s->attn_out);
	cudaFree(s->t);
	cudaFree(s->act);
	cudaFree(s->xnorm);
	cudaFree(s->logits);
	cudaFree(s->partial);
	cudaFree(s->tickets);
	cudaFree(s->attn_tickets);
	cudaFree(s->attn_part);
	cudaFree(s->step_pos);
	cudaFree(s->next_pos);
	cudaFree(s->ring_base);
	cudaFree(s->tok_log);
	cudaFree(s->force_ids);
	if (!s->randf_in_blk) cudaFree(s->randf);
	cudaFree(s->step_blk);  // err_flag, tok, randf_count, log_count (and the first randf)
	cudaFree(s->pf);
	cudaFree(s->pf_ids);
	cudaFree(s->bx);
	cudaFree(s->bup);
	cudaFree(s->btc.apack);
	cudaFree(s->btc.partial);
	cudaFree(s->btc.tickets);
	cudaFree(s->d_tmaps);
	cudaFree(s->d_layers);
	cudaFree(s->mg_ll);
	cudaFree(s->mg_probs);
	cudaFree(s->mg_pe);
	cudaFree(s->mg_samp_f);
	cudaFree(s->mg_samp_i);
	cudaFree(s->mg_bar);
	cudaFree(s->mg_dbg);
	cudaFree(s->d_pslayers);
	cudaFree(s->ps_ll);
	if (s->host_pin) cudaFreeHost(s->host_pin);
	if (s->stream) cudaStreamDestroy(s->stream);
	delete s;
	return TG_OK;
}

int tg_state_reset(tg_state *s) {
	if (!s) return fail(TG_EINVAL, "null state");
	TG_CUDA(cudaSetDevice(s->m->device));
	const int B = s->B;
	TG_CUDA(cudaMemsetAsync(s->step_pos, 0, 4 * B, s->stream));
	TG_CUDA(cudaMemsetAsync(s->next_pos, 0, 4 * B, s->stream));
	TG_CUDA(cudaMemsetAsync(s->ring_base, 0, 4 * B, s->stream));
	TG_CUDA(cudaMemsetAsync(s->log_count, 0, 4 * B, s->stream));
	TG_CUDA(cudaMemsetAsync(s->randf_count, 0, 4 * B, s->stream));
	TG_CUDA(cudaMemsetAsync(s->err_flag, 0, 4, s->stream));
	// the reference's caches are zero-initialised (tensor.hpp:66-74); stale rows
	// are never read (valid_pos bounds every loop) so they are left in place
	TG_CUDA(cudaStreamSynchronize(s->stream));
	s->host_pos.assign(B, 0);
	return TG_OK;
}

int tg_state_position(tg_state *s, int b, int *position) {
	if (!s || !position || b < 0 || b >= s->B) return fail(TG_EINVAL, "bad argument");
	*position = s->host_pos[b];
	return TG_OK;
}

int tg_state_stream(tg_state *s, void **stream) {
	if (!s || !stream) return fail(TG_EINVAL, "null argument");
	*stream = (void *)s->stream;
	return TG_OK;
}

int tg_prefill(tg_state *s, const int *ids, int S, float *logits_host) {
	if (!s || !ids || S < 1) return fail(TG_EINVAL, "bad argument");
	tg_model *m = s->m;
	TG_TRY(check_ready(m));
	const tg_config &c = m->cfg;
	if (S > c.n_pos) return fail(TG_EINVAL, "prompt longer than n_pos");
	if (S > s->max_pos_global) return fail(TG_EINVAL, "prompt longer than max_pos_global");
	for (int b = 0; b < s->B; b++)
		if (s->host_pos[b] != 0) return fail(TG_ESTATE, "prefill needs an empty KV cache (decode.hpp:78-79)");
	TG_CUDA(cudaSetDevice(m->device));
	const int D = c.hidden_size, I = c.intermediate_size, V = c.n_vocab;
	const int qd = c.n_head * c.head_dim, kd = c.n_kv * c.head_dim;
	if (S == 1) {
		// a one-token prompt takes the reference's decode branch (modules.hpp:135)
		TG_TRY(tg_decode(s, ids, logits_host));
		return TG_OK;
	}
	// Batches that take the batched decode step prefill their prompts together, up to 16384 rows per pass (the
	// scratch grows with the rows: 79 KB per row at the 1B shape); smaller batches stay one sequence per pass, so
	// that a sequence's results do not depend on its neighbours' presence.
	const int group = (s->batched_ok && env_int("TG_GEMM_TC", 1) && env_int("TG_PREFILL_GROUP", 1)) ? std::max(1, std::min(s->B, 16384 / S)) : 1;
	const size_t R = size_t(group) * S;  // rows per pass
	size_t need = R * (3 * size_t(D) + 2 * qd + 2 * kd + 2 * size_t(I));
	size_t part = std::max(size_t(4) * R * D, size_t(1) << 22);  // split-K scratch
	part = std::max(part, std::min(size_t(24) * R * std::max(I, qd), size_t(1) << 28));  // tensor-core GEMM partial sums (<= 1 GiB)
	need += part;
	need += (tc_pack_bytes(int(R), std::max(I, std::max(D, qd))) + 3) / 4 + 64;
	need += (attn_tc_plan(S).total() + 3) / 4 + 512;  // packed q, k, v of the tensor-core attention (long prompts)
	if (need > s->pf_floats) {
		if (s->pf) cudaFree(s->pf);
		s->pf = nullptr;
		s->pf_floats = 0;
		cudaError_t e = cudaMalloc(&s->pf, need * 4);
		if (e != cudaSuccess) return fail(TG_ENOMEM, std::string("cudaMalloc(prefill scratch): ") + cudaGetErrorString(e));
		s->pf_floats = need;
	}
	if (S * s->B > s->pf_ids_cap) {
		if (s->pf_ids) cudaFree(s->pf_ids);
		s->pf_ids = nullptr;
		TG_CUDA(cudaMalloc(&s->pf_ids, size_t(S) * s->B * 4));
		s->pf_ids_cap = S * s->B;
	}
	TG_CUDA(cudaMemcpyAsync(s->pf_ids, ids, size_t(S) * s->B * 4, cudaMemcpyHostToDevice, s->stream));
	for (int b = 0; b < s->B; b += group) TG_TRY(enqueue_prefill_seq(s, b, S, std::min(group, s->B - b)));
	// position_ptr = S; ring base per decode.hpp:98-103
	std::vector<int> pos(s->B, S), rb(s->B, S >= c.n_pos_local ? S : 0);
	TG_TRY(staging_acquire(s));
	std::memcpy(s->host_pin, pos.data(), 4 * s->B);
	std::memcpy(s->host_pin + s->B, rb.data(), 4 * s->B);
	TG_CUDA(cudaMemcpyAsync(s->next_pos, s->host_pin, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	TG_CUDA(cudaMemcpyAsync(s->step_pos, s->host_pin, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	TG_CUDA(cudaMemcpyAsync(s->ring_base, s->host_pin + s->B, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	if (logits_host)
		TG_CUDA(cudaMemcpyAsync(logits_host, s->logits, size_t(s->B) * V * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_TRY(check_err_flag(s));
	s->host_pos.assign(s->B, S);
	return TG_OK;
}

int tg_decode(tg_state *s, const int *ids, float *logits_host) {
	if (!s) return fail(TG_EINVAL, "null state");
	tg_model *m = s->m;
	TG_TRY(check_ready(m));
	TG_CUDA(cudaSetDevice(m->device));
	for (int b = 0; b < s->B; b++)
		if (s->host_pos[b] >= s->max_pos_global) return fail(TG_ESTATE, "global KV cache full (max_pos_global reached)");
	if (ids) {
		for (int b = 0; b < s->B; b++)
			if (ids[b] < 0 || ids[b] >= m->cfg.n_vocab) return fail(TG_EINVAL, "token id out of range");
		TG_TRY(staging_acquire(s));
		std::memcpy(s->host_pin, ids, 4 * s->B);
		TG_CUDA(cudaMemcpyAsync(s->tok, s->host_pin, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	}
	if (s->mega_ok)
		TG_TRY(mega_launch(s, 1, 0, 2.0f, 1.0f, false));
	else
		TG_TRY(enqueue_decode_step(s));
	for (int b = 0; b < s->B; b++) s->host_pos[b] += 1;
	s->staging_busy = s->staging_busy || ids != nullptr;  // (an earlier asynchronous call's copy may still be queued)
	if (logits_host) {
		TG_CUDA(cudaMemcpyAsync(logits_host, s->logits, size_t(s->B) * m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, s->stream));
		TG_TRY(check_err_flag(s));
	}
	// without a host read-back the call only enqueues: the step runs while the caller prepares the sampler
	// call, and a device-side error (a wait that ran out) is reported by the next call that synchronises
	return TG_OK;
}

int tg_append(tg_state *s, const int *ids, int n, float *logits_host) {
	if (!s || !ids || n < 1) return fail(TG_EINVAL, "bad argument");
	if (s->B != 1) return fail(TG_EINVAL, "tg_append: one sequence per state");
	tg_model *m = s->m;
	TG_TRY(check_ready(m));
	TG_CUDA(cudaSetDevice(m->device));
	if (s->host_pos[0] + n > s->max_pos_global) return fail(TG_ESTATE, "global KV cache too small for the appended tokens");
	for (int i = 0; i < n; i++)
		if (ids[i] < 0 || ids[i] >= m->cfg.n_vocab) return fail(TG_EINVAL, "token id out of range");
	if (s->ps_ok) {
		// one launch of the persistent kernel: every step takes its token from the list instead of a sampler
		if (s->force_cap < n) {
			cudaFree(s->force_ids);
			s->force_ids = nullptr;
			TG_CUDA(cudaMalloc(&s->force_ids, size_t(n) * 4));
			s->force_cap = n;
		}
		TG_CUDA(cudaMemcpyAsync(s->force_ids, ids, size_t(n) * 4, cudaMemcpyHostToDevice, s->stream));
		TG_CUDA(cudaStreamSynchronize(s->stream));  // `ids` is the caller's pageable memory: consumed before returning
		TG_TRY(persist_launch(s, n, 0, 2.0f, 1.0f, false, s->force_ids));
		s->host_pos[0] += n;
	} else {
		for (int i = 0; i < n; i++) TG_TRY(tg_decode(s, ids + i, nullptr));
	}
	if (logits_host)
		TG_CUDA(cudaMemcpyAsync(logits_host, s->logits, size_t(m->cfg.n_vocab) * 4, cudaMemcpyDeviceToHost, s->stream));
	return check_err_flag(s);
}

int tg_sample_argmax(tg_state *s, int *toks_host) {
	if (!s) return fail(TG_EINVAL, "null state");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_TRY(enqueue_sampler(s, 2.0f, 1.0f, false));
	TG_CUDA(cudaMemcpyAsync(s->host_pin, s->tok, 4 * s->B, cudaMemcpyDeviceToHost, s->stream));
	TG_TRY(check_err_flag(s));  // synchronises
	if (toks_host) std::memcpy(toks_host, s->host_pin, 4 * s->B);
	return TG_OK;
}

int tg_state_set_randf(tg_state *s, const float *randf_host, int n) {
	if (!s || !randf_host || n < 1) return fail(TG_EINVAL, "bad argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	if (n > s->randf_cap) {
		if (s->randf && !s->randf_in_blk) cudaFree(s->randf);
		s->randf = nullptr;
		s->randf_in_blk = false;
		s->randf_cap = 0;
		TG_CUDA(cudaMalloc(&s->randf, size_t(n) * s->B * 4));
		s->randf_cap = n;
		// captured graphs do not hold this pointer (the sampler is launched outside the graph)
	}
	TG_CUDA(cudaMemcpyAsync(s->randf, randf_host, size_t(n) * s->B * 4, cudaMemcpyHostToDevice, s->stream));
	TG_CUDA(cudaMemsetAsync(s->randf_count, 0, 4 * s->B, s->stream));
	TG_CUDA(cudaStreamSynchronize(s->stream));
	s->randf_valid = std::max(s->randf_valid, n);
	return TG_OK;
}

int tg_sample_minp(tg_state *s, float minp, float temp, const float *randf_host, int *toks_host) {
	if (!s || !randf_host) return fail(TG_EINVAL, "bad argument");
	if (!(minp < 1.0f)) return fail(TG_EINVAL, "minp must be < 1 (the reference uses argmax otherwise, transformer.hpp:208)");
	TG_CUDA(cudaSetDevice(s->m->device));
	if (s->randf_cap >= 1 && size_t(s->B) * 4 <= 4096) {
		// one uniform per sequence, staged through pinned memory: no synchronisation before the launch
		s->randf_valid = std::max(s->randf_valid, 1);
		float *stage = reinterpret_cast<float *>(s->host_pin + 4096);
		std::memcpy(stage, randf_host, size_t(s->B) * 4);
		TG_CUDA(cudaMemcpyAsync(s->randf, stage, size_t(s->B) * 4, cudaMemcpyHostToDevice, s->stream));
		TG_CUDA(cudaMemsetAsync(s->randf_count, 0, 4 * s->B, s->stream));
	} else {
		TG_TRY(tg_state_set_randf(s, randf_host, 1));
	}
	TG_TRY(enqueue_sampler(s, minp, temp, false));
	TG_CUDA(cudaMemcpyAsync(s->host_pin, s->tok, 4 * s->B, cudaMemcpyDeviceToHost, s->stream));
	TG_TRY(check_err_flag(s));  // synchronises
	if (toks_host) std::memcpy(toks_host, s->host_pin, 4 * s->B);
	return TG_OK;
}

int tg_logits_read(tg_state *s, float *logits_host) {
	if (!s || !logits_host) return fail(TG_EINVAL, "null argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_CUDA(cudaMemcpyAsync(logits_host, s->logits, size_t(s->B) * s->m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_CUDA(cudaStreamSynchronize(s->stream));
	return TG_OK;
}

namespace {
// `counters_zeroed`: the caller's upload has already set log_count (and randf_count) to zero
int generate_async(tg_state *s, int n_steps, float minp, float temp, bool counters_zeroed) {
	TG_TRY(check_ready(s->m));
	TG_CUDA(cudaSetDevice(s->m->device));
	if (s->host_pos[0] + n_steps > s->max_pos_global) return fail(TG_ESTATE, "global KV cache too small for n_steps");
	if (minp < 1.0f && s->randf_valid < n_steps) return fail(TG_ESTATE, "upload uniforms first (tg_state_set_randf)");
	TG_TRY(ensure_log(s, n_steps));
	if (!counters_zeroed) TG_CUDA(cudaMemsetAsync(s->log_count, 0, 4 * s->B, s->stream));
	if (s->mega_ok) {
		TG_TRY(mega_launch(s, n_steps, minp < 1.0f ? 2 : 1, minp, temp, true));
	} else {
		for (int i = 0; i < n_steps; i++) {
			TG_TRY(enqueue_decode_step(s));
			TG_TRY(enqueue_sampler(s, minp, temp, true));
		}
	}
	for (int b = 0; b < s->B; b++) s->host_pos[b] += n_steps;
	return TG_OK;
}
}  // namespace

int tg_generate_async(tg_state *s, int n_steps, float minp, float temp) {
	if (!s || n_steps < 1) return fail(TG_EINVAL, "bad argument");
	return generate_async(s, n_steps, minp, temp, false);
}

int tg_state_tokens(tg_state *s, int n_steps, int *toks_host) {
	if (!s || !toks_host || n_steps < 1 || n_steps > s->log_cap) return fail(TG_EINVAL, "bad argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_CUDA(cudaMemcpyAsync(toks_host, s->tok_log, size_t(n_steps) * s->B * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_TRY(check_err_flag(s));
	return TG_OK;
}

int tg_generate(tg_state *s, const int *first_ids, int n_steps, float minp, float temp, const float *randf_host,
                int *toks_host) {
	if (!s || !first_ids || n_steps < 1) return fail(TG_EINVAL, "bad argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	// Short runs (a step at a time from a host loop) go through the pinned staging buffer with one
	// synchronisation at the end: ids and uniforms in, the launch, tokens out.
	const size_t nbytes = size_t(n_steps) * s->B * 4;
	const bool lean = nbytes <= 16384;
	TG_TRY(staging_acquire(s));
	if (minp < 1.0f && !randf_host) return fail(TG_EINVAL, "min-p sampling needs uniforms");
	if (n_steps == 1 && s->B == 1 && s->ps_ok && env_int("TG_LEAN_STEP", 1)) {
		// One token per call (a host loop around the sampler): the step's inputs — id, uniform, zeroed
		// counters — lie next to each other in the state's step block and go up in ONE copy; the error word
		// and the sampled id lie next to each other too and come back in ONE; the persistent kernel leaves
		// its arena and barrier ready for the next launch. So the call is upload, launch, read-back, wait.
		if (first_ids[0] < 0 || first_ids[0] >= s->m->cfg.n_vocab) return fail(TG_EINVAL, "token id out of range");
		int *up = s->host_pin;
		up[0] = first_ids[0];  // tok
		up[1] = 0;             // randf_count
		up[2] = 0;             // log_count
		if (minp < 1.0f) {
			std::memcpy(up + 3, randf_host, 4);
			s->randf_valid = std::max(s->randf_valid, 1);
		}
		TG_CUDA(cudaMemcpyAsync(s->tok, up, minp < 1.0f ? 16 : 12, cudaMemcpyHostToDevice, s->stream));
		s->lean_randf = true;
		const int rc = generate_async(s, 1, minp, temp, true);
		s->lean_randf = false;
		if (rc) return rc;
		int *down = s->host_pin + 8192;
		TG_CUDA(cudaMemcpyAsync(down, s->err_flag, 20, cudaMemcpyDeviceToHost, s->stream));  // err_flag, pad, tok
		TG_CUDA(cudaStreamSynchronize(s->stream));
		s->staging_busy = false;
		TG_TRY(report_err_flag(s, down[0]));
		if (toks_host) toks_host[0] = down[4];
		return TG_OK;
	}
	if (minp < 1.0f) {
		if (lean && s->randf_cap >= n_steps) {
			s->randf_valid = std::max(s->randf_valid, n_steps);
			float *stage = reinterpret_cast<float *>(s->host_pin + 4096);
			std::memcpy(stage, randf_host, nbytes);
			TG_CUDA(cudaMemcpyAsync(s->randf, stage, nbytes, cudaMemcpyHostToDevice, s->stream));
			TG_CUDA(cudaMemsetAsync(s->randf_count, 0, 4 * s->B, s->stream));
		} else {
			TG_TRY(tg_state_set_randf(s, randf_host, n_steps));
		}
	}
	for (int b = 0; b < s->B; b++)
		if (first_ids[b] < 0 || first_ids[b] >= s->m->cfg.n_vocab) return fail(TG_EINVAL, "token id out of range");
	std::memcpy(s->host_pin, first_ids, 4 * s->B);
	TG_CUDA(cudaMemcpyAsync(s->tok, s->host_pin, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	TG_TRY(tg_generate_async(s, n_steps, minp, temp));
	if (toks_host && lean) {
		// (stream order: the ids above were consumed by their copy before this one writes the buffer)
		TG_CUDA(cudaMemcpyAsync(s->host_pin, s->tok_log, nbytes, cudaMemcpyDeviceToHost, s->stream));
		TG_TRY(check_err_flag(s));  // synchronises
		std::memcpy(toks_host, s->host_pin, nbytes);
		return TG_OK;
	}
	if (toks_host) return tg_state_tokens(s, n_steps, toks_host);
	TG_CUDA(cudaStreamSynchronize(s->stream));
	return TG_OK;
}

int tg_kv_read(tg_state *s, int b, int layer, int slot0, int nslots, float *k_host, float *v_host) {
	if (!s || !k_host || !v_host || b < 0 || b >= s->B || layer < 0 || layer >= s->m->cfg.n_layers)
		return fail(TG_EINVAL, "bad argument");
	const int slots = s->slots[layer];
	if (slot0 < 0 || nslots < 1 || slot0 + nslots > slots) return fail(TG_EINVAL, "slot range out of bounds");
	TG_CUDA(cudaSetDevice(s->m->device));
	size_t off = (size_t(b) * slots + slot0) * AT_HD;
	TG_CUDA(cudaMemcpyAsync(k_host, s->kcache[layer] + off, size_t(nslots) * AT_HD * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_CUDA(cudaMemcpyAsync(v_host, s->vcache[layer] + off, size_t(nslots) * AT_HD * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_CUDA(cudaStreamSynchronize(s->stream));
	return TG_OK;
}

int tg_hidden_read(tg_state *s, float *hidden_host) {
	if (!s || !hidden_host) return fail(TG_EINVAL, "null argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_CUDA(cudaMemcpyAsync(hidden_host, s->xnorm, size_t(s->B) * s->m->cfg.hidden_size * 4, cudaMemcpyDeviceToHost, s->stream));
	TG_CUDA(cudaStreamSynchronize(s->stream));
	return TG_OK;
}

// ---------------------------------------------------------------- vocab-sharded lm_head support
int tg_decode_hidden(tg_state *s, const int *ids) {
	if (!s) return fail(TG_EINVAL, "null state");
	tg_model *m = s->m;
	TG_TRY(check_ready(m));
	TG_CUDA(cudaSetDevice(m->device));
	for (int b = 0; b < s->B; b++)
		if (s->host_pos[b] >= s->max_pos_global) return fail(TG_ESTATE, "global KV cache full (max_pos_global reached)");
	if (ids) {
		TG_TRY(staging_acquire(s));
		std::memcpy(s->host_pin, ids, 4 * s->B);
		TG_CUDA(cudaMemcpyAsync(s->tok, s->host_pin, 4 * s->B, cudaMemcpyHostToDevice, s->stream));
	}
	if (s->batched_ok) {
		TG_TRY(enqueue_decode_batched(s, false));
	} else {
		for (int b0 = 0; b0 < s->B; b0 += MV_MAX_B) TG_TRY(enqueue_decode_chunk(s, b0, std::min(MV_MAX_B, s->B - b0), false));
	}
	if (ids) TG_TRY(check_err_flag(s));  // fed from the device: enqueue only, tg_state_check reports the error word later
	for (int b = 0; b < s->B; b++) s->host_pos[b] += 1;
	return TG_OK;
}

int tg_state_check(tg_state *s) {
	if (!s) return fail(TG_EINVAL, "null state");
	TG_CUDA(cudaSetDevice(s->m->device));
	return check_err_flag(s);
}

int tg_dev_hidden_copy(tg_state *s, float *dst_dev) {
	if (!s || !dst_dev) return fail(TG_EINVAL, "null argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_CUDA(cudaMemcpyAsync(dst_dev, s->xnorm, size_t(s->B) * s->m->cfg.hidden_size * 4, cudaMemcpyDeviceToDevice, s->stream));
	return TG_OK;
}

int tg_dev_set_tokens(tg_state *s, const int *toks_dev) {
	if (!s || !toks_dev) return fail(TG_EINVAL, "null argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	TG_CUDA(cudaMemcpyAsync(s->tok, toks_dev, size_t(s->B) * 4, cudaMemcpyDeviceToDevice, s->stream));
	return TG_OK;
}

int tg_dev_lm_head_top1(tg_model *m, const float *hidden_dev, int M, int col0, int ncols, float *max_dev, int *idx_dev,
                        void *stream) {
	if (!m || !hidden_dev || !max_dev || !idx_dev || M < 1) return fail(TG_EINVAL, "bad argument");
	const int V = m->cfg.n_vocab, D = m->cfg.hidden_size;
	if (col0 < 0 || ncols < MV_TN || col0 % MV_TN || ncols % MV_TN || col0 + ncols > V)
		return fail(TG_EINVAL, "vocabulary slice must be a multiple of 128 columns inside [0, n_vocab)");
	TG_CUDA(cudaSetDevice(m->device));
	cudaStream_t st = (cudaStream_t)stream;
	// One tensor-core GEMM over the slice, addressed in place through a tensor map with the full matrix's row
	// pitch (a tile row is a 128- or 256-byte segment either way); its epilogue keeps per row the largest
	// scaled value and its column, so no logits are written. Scratch per device, grown on demand.
	struct Top1Scratch {
		TcScratch tc;
		unsigned long long *keys = nullptr;
		int keys_cap = 0;
		int *err_host = nullptr;
	};
	static Top1Scratch scr[TG_MAX_DEVICES];
	const int slot = current_device_slot();
	Top1Scratch &t = scr[slot];
	const size_t need = tc_pack_bytes(M, D);
	if (need > t.tc.apack_bytes) {
		if (t.tc.apack) cudaFree(t.tc.apack);
		t.tc.apack = nullptr;
		t.tc.apack_bytes = 0;
		TG_CUDA(cudaMalloc(&t.tc.apack, need));
		t.tc.apack_bytes = need;
	}
	if (M > t.keys_cap) {
		if (t.keys) cudaFree(t.keys);
		t.keys = nullptr;
		t.keys_cap = 0;
		TG_CUDA(cudaMalloc(&t.keys, size_t(M) * 8));
		t.keys_cap = M;
	}
	if (!t.tc.err) {
		TG_CUDA(cudaMalloc(&t.tc.err, 4));
		TG_CUDA(cudaMemset(t.tc.err, 0, 4));
		TG_CUDA(cudaHostAlloc(&t.err_host, 4, cudaHostAllocDefault));
		*t.err_host = 0;
	}
	// The call only enqueues. The GEMM's error word is copied out behind it and looked at by the next call on
	// this device (a wait that ran out shows up one call late instead of costing a synchronisation per step).
	if (*static_cast<volatile int *>(t.err_host)) {
		*t.err_host = 0;
		cudaMemsetAsync(t.tc.err, 0, 4, st);
		return fail(TG_ECUDA, "tensor-core GEMM: a pipeline wait ran out in an earlier tg_dev_lm_head_top1 on this device");
	}
	TG_CUDA(cudaMemsetAsync(t.keys, 0, size_t(M) * 8, st));
	TG_TRY(pack_activations(hidden_dev, M, D, t.tc, st));
	QW slice{m->lm_head.q + col0, m->lm_head.s + col0, D, ncols, V};
	TcScratch one = t.tc;
	one.top1 = t.keys;
	one.top1_col0 = col0;
	float *Cs[1] = {nullptr};
	const QW *ws[1] = {&slice};
	TG_TRY(launch_gemm_tc_group(1, Cs, ws, nullptr, M, one, st, 1));
	top1_unpack_kernel<<<(M + 127) / 128, 128, 0, st>>>(t.keys, M, max_dev, idx_dev);
	count_launch();
	TG_TRY(check_launch("top1_unpack"));
	TG_CUDA(cudaMemcpyAsync(t.err_host, t.tc.err, 4, cudaMemcpyDeviceToHost, st));
	return TG_OK;
}

// gathered candidates [world][2][M] (row 0: maxima as fp32 bits, row 1: global indices) -> tokens of rows
// row0 .. row0 + nrows: the largest maximum, among equal maxima the lowest index (the tie rule of
// ops::argmax_logits, reference ops.hpp:744-760); a slice without a candidate (index -1) never wins; -1 if none has one
__global__ void resolve_top1_kernel(const int *cand, int world, int M, int row0, int nrows, int *toks) {
	const int r = blockIdx.x * blockDim.x + threadIdx.x;
	if (r >= nrows) return;
	float best = -INFINITY;
	int arg = -1;
	for (int w = 0; w < world; w++) {
		const float v = __int_as_float(cand[(size_t(w) * 2) * M + row0 + r]);
		const int i = cand[(size_t(w) * 2 + 1) * M + row0 + r];
		if (i < 0) continue;
		if (arg < 0 || v > best || (v == best && i < arg)) {
			best = v;
			arg = i;
		}
	}
	toks[r] = arg;
}

int tg_dev_resolve_top1(const void *cand_all_dev, int world, int M, int row0, int nrows, int *toks_dev, void *stream) {
	if (!cand_all_dev || !toks_dev || world < 1 || M < 1 || row0 < 0 || nrows < 1 || row0 + nrows > M)
		return fail(TG_EINVAL, "bad argument");
	resolve_top1_kernel<<<(nrows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(static_cast<const int *>(cand_all_dev), world, M, row0, nrows, toks_dev);
	count_launch();
	return check_launch("resolve_top1");
}

// ---------------------------------------------------------------- isolated ops
int tg_dev_qmatvec(float *y, const float *x, const int8_t *w, const float *scales, int K, int N, void *stream) {
	if (!y || !x || !w || !scales) return fail(TG_EINVAL, "null argument");
	if (!supported_k(K)) return fail(TG_ESHAPE, "Unsupported ROW dimension: " + std::to_string(K));
	if (!supported_n(N)) return fail(TG_ESHAPE, "Unsupported COL dimension: " + std::to_string(N));
	// scratch for split-K, per device, grown on demand
	static float *partial[64] = {nullptr};
	static size_t partial_floats[64] = {0};
	static unsigned *tickets[64] = {nullptr};
	int dev = 0;
	TG_CUDA(cudaGetDevice(&dev));
	int sms = 0;
	if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) g_num_sms = sms;
	// the layer matrices: one wave of CTAs, K split over a thread-block cluster (TG_MV_CLUSTER=0: the split-K kernel below)
	if (env_int("TG_MV_CLUSTER", 1)) {
		const MvcPlan cp = mvc_plan(K, N, dev);
		if (cp.ks) return mvc_launch(cp, y, x, w, scales, K, N, (cudaStream_t)stream);
	}
	// K-split depth capped (measured on the isolated operator: deeper splits only lengthen the last CTA's sum)
	MvPlan p = plan_matvec(K, N / MV_TN, env_int("TG_MV_TARGET_CTAS", 2 * g_num_sms), env_int("TG_MV_MAX_SPLIT", K >= 4096 ? 32 : 16));
	size_t need = size_t(p.nsplit) * N;
	if (need > partial_floats[dev]) {
		if (partial[dev]) cudaFree(partial[dev]);
		partial[dev] = nullptr;
		TG_CUDA(cudaMalloc(&partial[dev], need * 4));
		partial_floats[dev] = need;
	}
	if (!tickets[dev]) {
		TG_CUDA(cudaMalloc(&tickets[dev], sizeof(unsigned) * 2048));
		TG_CUDA(cudaMemset(tickets[dev], 0, sizeof(unsigned) * 2048));
	}
	MvArgs a{};
	a.seg[0] = MvSeg{w, scales, N, 0, 0};
	a.nseg = 1;
	a.ntiles = N / MV_TN;
	a.K = K;
	a.kc = p.kc;
	a.nsplit = p.nsplit;
	a.B = 1;
	a.part_stride = N;
	a.out_stride = N;
	a.x = x;
	a.partial = partial[dev];
	a.tickets = tickets[dev];
	a.out = y;
	return launch_mv(a, PRO_PLAIN, EPI_SCALE, (cudaStream_t)stream);
}

// ---------------------------------------------------------------- matvec that allocates nothing
// Some hosts of this library must not call cudaMalloc on the request path: a
// serving process that pre-reserves all of HBM for its own pools, a real-time
// loop that cannot take the allocator's implicit device synchronisation, or code
// that runs while a stream is being captured into a CUDA graph, where cudaMalloc
// is illegal. tg_dev_qmatvec grows two device buffers on demand (split-K partial
// sums and column-tile tickets); this variant keeps them in the fixed array
// below instead. The array is part of the library image: every GPU that loads
// the library holds these 264 KiB until the process exits.
constexpr int STATIC_MAX_TILES = 2048;                 // N <= 262144 columns
constexpr size_t STATIC_PARTIAL_FLOATS = 64 * 1024;    // nsplit * N <= 65536 partial sums
constexpr size_t STATIC_TICKET_BYTES = STATIC_MAX_TILES * sizeof(unsigned);
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_TICKET_BYTES + STATIC_PARTIAL_FLOATS * sizeof(float)];

int tg_dev_qmatvec_static(float *y, const float *x, const int8_t *w, const float *scales, int K, int N, void *stream) {
	if (!y || !x || !w || !scales) return fail(TG_EINVAL, "null argument");
	if (N > STATIC_MAX_TILES * MV_TN)
		return fail(TG_EINVAL, "N = " + std::to_string(N) + " is beyond the static scratch maximum of " +
		                           std::to_string(STATIC_MAX_TILES * MV_TN) + " columns");
	if (!supported_k(K)) return fail(TG_ESHAPE, "Unsupported ROW dimension: " + std::to_string(K));
	if (!supported_n(N)) return fail(TG_ESHAPE, "Unsupported COL dimension: " + std::to_string(N));
	// Set-up, once per device and with that device current: in host code the array's name is only
	// a stand-in for the device symbol, so its device address is asked for here and that pointer
	// is what the kernel gets. This first call per device should come before any stream capture.
	static unsigned char *scratch_dev[64] = {nullptr};
	static int sms_dev[64] = {0};
	int dev = 0;
	TG_CUDA(cudaGetDevice(&dev));
	if (dev < 0 || dev >= 64) return fail(TG_EINVAL, "device index out of range");
	if (!scratch_dev[dev]) {
		unsigned char *ptr = nullptr;
		cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
		if (e != cudaSuccess || !ptr) return fail(TG_ECUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
		int sms = 0;
		TG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
		sms_dev[dev] = sms > 0 ? sms : 148;
		scratch_dev[dev] = ptr;
	}
	g_num_sms = sms_dev[dev];
	// the K-split is capped so that the partial sums fit the fixed array
	const int max_split = int(STATIC_PARTIAL_FLOATS / size_t(N)) > 0 ? int(STATIC_PARTIAL_FLOATS / size_t(N)) : 1;
	MvPlan p = plan_matvec(K, N / MV_TN, 2 * g_num_sms, max_split);
	if (p.nsplit > 1 && size_t(p.nsplit) * N > STATIC_PARTIAL_FLOATS)
		return fail(TG_EINVAL, "split-K partial sums exceed the static scratch maximum of " +
		                           std::to_string(STATIC_PARTIAL_FLOATS) + " floats");
	unsigned *tickets = reinterpret_cast<unsigned *>(scratch_dev[dev]);
	float *partial = reinterpret_cast<float *>(scratch_dev[dev] + STATIC_TICKET_BYTES);
	// every call shares the array and finds the previous call's contents in it: the tickets must
	// start at zero (the partial sums are fully overwritten before they are read)
	TG_CUDA(cudaMemsetAsync(tickets, 0, sizeof(unsigned) * size_t(N / MV_TN), (cudaStream_t)stream));
	MvArgs a{};
	a.seg[0] = MvSeg{w, scales, N, 0, 0};
	a.nseg = 1;
	a.ntiles = N / MV_TN;
	a.K = K;
	a.kc = p.kc;
	a.nsplit = p.nsplit;
	a.B = 1;
	a.part_stride = N;
	a.out_stride = N;
	a.x = x;
	a.partial = partial;
	a.tickets = tickets;
	a.out = y;
	return launch_mv(a, PRO_PLAIN, EPI_SCALE, (cudaStream_t)stream);
}

int tg_dev_qgemm(float *c, const float *a, const int8_t *w, const float *scales, int M, int K, int N, void *stream) {
	if (!c || !a || !w || !scales || M < 1) return fail(TG_EINVAL, "bad argument");
	if (!supported_k(K)) return fail(TG_ESHAPE, "Unsupported ROW dimension: " + std::to_string(K));
	if (!supported_n(N)) return fail(TG_ESHAPE, "Unsupported COL dimension: " + std::to_string(N));
	int dev = 0;
	TG_CUDA(cudaGetDevice(&dev));
	QW q{w, scales, K, N};
	if (env_int("TG_GEMM_TC", 1)) {
		// tensor-core path: packed bf16 activations + an error word, per device, grown on demand
		static TcScratch tc[64];
		const size_t need = tc_pack_bytes(M, K);
		if (need > tc[dev].apack_bytes) {
			if (tc[dev].apack) cudaFree(tc[dev].apack);
			tc[dev].apack = nullptr;
			tc[dev].apack_bytes = 0;
			TG_CUDA(cudaMalloc(&tc[dev].apack, need));
			tc[dev].apack_bytes = need;
		}
		const size_t pneed = std::min(size_t(24) * M * N, size_t(1) << 28);
		if (pneed > tc[dev].partial_floats) {
			if (tc[dev].partial) cudaFree(tc[dev].partial);
			tc[dev].partial = nullptr;
			tc[dev].partial_floats = 0;
			TG_CUDA(cudaMalloc(&tc[dev].partial, pneed * 4));
			tc[dev].partial_floats = pneed;
		}
		if (!tc[dev].err) {
			TG_CUDA(cudaMalloc(&tc[dev].err, 4));
			TG_CUDA(cudaMemset(tc[dev].err, 0, 4));
		}
		TG_TRY(pack_activations(a, M, K, tc[dev], (cudaStream_t)stream));
		TG_TRY(launch_gemm_tc(c, q, M, tc[dev], (cudaStream_t)stream));
		// while the stream is being captured into a graph nothing may synchronise: the error word stays
		// set on the device and the next call outside a capture reports it
		cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
		TG_CUDA(cudaStreamIsCapturing((cudaStream_t)stream, &cap));
		if (cap != cudaStreamCaptureStatusNone) return TG_OK;
		int flag = 0;
		TG_CUDA(cudaMemcpyAsync(&flag, tc[dev].err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
		TG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
		if (flag) {
			cudaMemset(tc[dev].err, 0, 4);
			return fail(TG_ECUDA, "tensor-core GEMM: a pipeline wait ran out");
		}
		return TG_OK;
	}
	static float *partial[64] = {nullptr};
	static size_t partial_floats[64] = {0};
	size_t need = std::max(size_t(4) * M * N, size_t(1) << 20);
	if ((N / GM_BN) * ((M + GM_BM - 1) / GM_BM) >= g_num_sms) need = 0;
	if (need > partial_floats[dev]) {
		if (partial[dev]) cudaFree(partial[dev]);
		partial[dev] = nullptr;
		TG_CUDA(cudaMalloc(&partial[dev], need * 4));
		partial_floats[dev] = need;
	}
	return launch_gemm(c, a, q, M, partial[dev], partial_floats[dev], (cudaStream_t)stream);
}

namespace {
struct DevBuf {
	void *p = nullptr;
	~DevBuf() {
		if (p) cudaFree(p);
	}
	int alloc(size_t n) {
		TG_CUDA(cudaMalloc(&p, n));
		return TG_OK;
	}
};
}  // namespace

int tg_qmatvec(float *y, const float *x, const int8_t *w, const float *scales, int K, int N) {
	if (!y || !x || !w || !scales) return fail(TG_EINVAL, "null argument");
	if (!supported_k(K)) return fail(TG_ESHAPE, "Unsupported ROW dimension: " + std::to_string(K));
	if (!supported_n(N)) return fail(TG_ESHAPE, "Unsupported COL dimension: " + std::to_string(N));
	TG_TRY(ensure_device(0));
	DevBuf dy, dx, dw, ds;
	TG_TRY(dy.alloc(size_t(N) * 4));
	TG_TRY(dx.alloc(size_t(K) * 4));
	TG_TRY(dw.alloc(size_t(K) * N));
	TG_TRY(ds.alloc(size_t(N) * 4));
	TG_CUDA(cudaMemcpy(dx.p, x, size_t(K) * 4, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(dw.p, w, size_t(K) * N, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(ds.p, scales, size_t(N) * 4, cudaMemcpyHostToDevice));
	TG_TRY(tg_dev_qmatvec((float *)dy.p, (const float *)dx.p, (const int8_t *)dw.p, (const float *)ds.p, K, N, nullptr));
	TG_CUDA(cudaDeviceSynchronize());
	TG_CUDA(cudaMemcpy(y, dy.p, size_t(N) * 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_qgemm(float *c, const float *a, const int8_t *w, const float *scales, int M, int K, int N) {
	if (!c || !a || !w || !scales || M < 1) return fail(TG_EINVAL, "bad argument");
	if (!supported_k(K)) return fail(TG_ESHAPE, "Unsupported ROW dimension: " + std::to_string(K));
	if (!supported_n(N)) return fail(TG_ESHAPE, "Unsupported COL dimension: " + std::to_string(N));
	TG_TRY(ensure_device(0));
	DevBuf dc, da, dw, ds;
	TG_TRY(dc.alloc(size_t(M) * N * 4));
	TG_TRY(da.alloc(size_t(M) * K * 4));
	TG_TRY(dw.alloc(size_t(K) * N));
	TG_TRY(ds.alloc(size_t(N) * 4));
	TG_CUDA(cudaMemcpy(da.p, a, size_t(M) * K * 4, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(dw.p, w, size_t(K) * N, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(ds.p, scales, size_t(N) * 4, cudaMemcpyHostToDevice));
	TG_TRY(tg_dev_qgemm((float *)dc.p, (const float *)da.p, (const int8_t *)dw.p, (const float *)ds.p, M, K, N, nullptr));
	TG_CUDA(cudaDeviceSynchronize());
	TG_CUDA(cudaMemcpy(c, dc.p, size_t(M) * N * 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_argmax_logits(const float *logits, int n, int *tok) {
	if (!logits || !tok || n < 4 || n % 4) return fail(TG_EINVAL, "bad argument (n must be a multiple of 4)");
	TG_TRY(ensure_device(0));
	DevBuf dl, dt, dc;
	TG_TRY(dl.alloc(size_t(n) * 4));
	TG_TRY(dt.alloc(4));
	TG_TRY(dc.alloc(4));
	TG_CUDA(cudaMemcpy(dl.p, logits, size_t(n) * 4, cudaMemcpyHostToDevice));
	SampleArgs a{};
	a.logits = (float *)dl.p;
	a.V = n;
	a.tok_out = (int *)dt.p;
	a.B = 1;
	argmax_kernel<<<1, SM_THREADS>>>(a);
	count_launch();
	TG_TRY(check_launch("argmax"));
	TG_CUDA(cudaMemcpy(tok, dt.p, 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_minp_logits(float *logits, int n, float minp, float temp, float randf, int *tok) {
	if (!logits || !tok || n < MP_CHUNK || n % MP_CHUNK) return fail(TG_EINVAL, "bad argument (n must be a multiple of 8192)");
	TG_TRY(ensure_device(0));
	DevBuf dl, dt, dr, dc;
	TG_TRY(dl.alloc(size_t(n) * 4));
	TG_TRY(dt.alloc(4));
	TG_TRY(dr.alloc(4));
	TG_TRY(dc.alloc(4));
	TG_CUDA(cudaMemcpy(dl.p, logits, size_t(n) * 4, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(dr.p, &randf, 4, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemset(dc.p, 0, 4));
	SampleArgs a{};
	a.logits = (float *)dl.p;
	a.V = n;
	a.tok_out = (int *)dt.p;
	a.B = 1;
	a.minp = minp;
	a.temp = temp;
	a.randf = (const float *)dr.p;
	a.randf_count = (int *)dc.p;
	a.randf_cap = 1;
	minp_kernel<<<1, SM_THREADS>>>(a);
	count_launch();
	TG_TRY(check_launch("minp"));
	TG_CUDA(cudaMemcpy(tok, dt.p, 4, cudaMemcpyDeviceToHost));
	TG_CUDA(cudaMemcpy(logits, dl.p, size_t(n) * 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_inverse_cdf(const float *p, int n, float cum0, float randf, int *idx, float *cum_out) {
	if (!p || !idx || n < 1) return fail(TG_EINVAL, "bad argument");
	TG_TRY(ensure_device(0));
	DevBuf dp, di, dc;
	TG_TRY(dp.alloc(size_t(n) * 4));
	TG_TRY(di.alloc(4));
	TG_TRY(dc.alloc(4));
	TG_CUDA(cudaMemcpy(dp.p, p, size_t(n) * 4, cudaMemcpyHostToDevice));
	inverse_cdf_kernel<<<1, SM_THREADS>>>((const float *)dp.p, n, cum0, randf, (int *)di.p, (float *)dc.p);
	count_launch();
	TG_TRY(check_launch("inverse_cdf"));
	TG_CUDA(cudaMemcpy(idx, di.p, 4, cudaMemcpyDeviceToHost));
	if (cum_out) TG_CUDA(cudaMemcpy(cum_out, dc.p, 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_rmsnorm(float *x, const float *w, int rows, int dim) {
	if (!x || !w || rows < 1 || dim < 1) return fail(TG_EINVAL, "bad argument");
	TG_TRY(ensure_device(0));
	DevBuf dx, dw;
	TG_TRY(dx.alloc(size_t(rows) * dim * 4));
	TG_TRY(dw.alloc(size_t(dim) * 4));
	TG_CUDA(cudaMemcpy(dx.p, x, size_t(rows) * dim * 4, cudaMemcpyHostToDevice));
	TG_CUDA(cudaMemcpy(dw.p, w, size_t(dim) * 4, cudaMemcpyHostToDevice));
	rmsnorm_rows_kernel<<<rows, 256>>>((float *)dx.p, (const float *)dx.p, (const float *)dw.p, nullptr, dim);
	count_launch();
	TG_TRY(check_launch("rmsnorm"));
	TG_CUDA(cudaMemcpy(x, dx.p, size_t(rows) * dim * 4, cudaMemcpyDeviceToHost));
	return TG_OK;
}

int tg_state_phase_clocks(tg_state *s, long long *clocks_host, int cap, int *n) {
	if (!s || !n) return fail(TG_EINVAL, "null argument");
	TG_CUDA(cudaSetDevice(s->m->device));
	if (!s->mg_dbg) {  // first call arms the recorder; later launches fill it
		TG_CUDA(cudaMalloc(&s->mg_dbg, 4096 * sizeof(long long)));
		TG_CUDA(cudaMemset(s->mg_dbg, 0, 4096 * sizeof(long long)));
		*n = 0;
		return TG_OK;
	}
	TG_CUDA(cudaStreamSynchronize(s->stream));
	std::vector<long long> tmp(4096);
	TG_CUDA(cudaMemcpy(tmp.data(), s->mg_dbg, 4096 * sizeof(long long), cudaMemcpyDeviceToHost));
	int k = 0;
	while (k < 4096 && tmp[k] != 0) k++;
	*n = k;
	if (clocks_host) std::memcpy(clocks_host, tmp.data(), sizeof(long long) * std::min(cap >= 4096 ? 4096 : k, cap));
	TG_CUDA(cudaMemset(s->mg_dbg, 0, 4096 * sizeof(long long)));
	return TG_OK;
}

int tg_launch_count(int reset, long long *count) {
	if (count) *count = g_launches.load();
	if (reset) g_launches.store(0);
	return TG_OK;
}

}  // extern "C"
