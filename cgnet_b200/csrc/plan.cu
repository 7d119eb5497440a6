// Plan construction (host side) and the Clebsch-Gordan table kernel.
//
// The plan replaces the seven int32 index tensors the reference keeps on its Python modules
// (CGNet/CG_layers.py:244-250 and :104-108) and the per-call constant uploads of its launchers
// (CGNet/cudaCG/cudaCG_sparse.cu:336-339): everything that depends only on (lmax, tau_in, tau_out, triples) is
// computed once here and stays resident on the device.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace cgb200 {

static thread_local std::string g_last_error;
// Launch accounting is process-wide: autograd runs the backward kernels on its own thread.
static std::atomic<int64_t> g_launches{0};
static std::mutex g_timing_mutex;

void set_error(const std::string& msg) { g_last_error = msg; }
int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string("CUDA error in ") + what + ": " + cudaGetErrorString(e);
    return CGB200_ERR_CUDA;
}

static const char* kKernelNames[K_COUNT] = {"cg_table", "cg_product_fwd", "cg_product_bwd", "fn_stats", "wmm_fwd",
                                            "wmm_bwd_w", "wmm_bwd_mid", "prep_transpose", "fused_stats", "fused_fwd",
                                            "fused_grad_w", "fused_grad_f", "fused_grad_f_reduce",
                                            "fused_grad_w_reduce", "tc_pack_weights", "fused_fwd_tensor", "fused_grad_w_tensor", "fused_grad_f_tensor",
                                            "sh_pack", "sh_project_tensor", "raycast_pack", "raycast_sphere", "fused_fwd_tensor_reduce", "grad_mid_pack_weights",
                                            "grad_mid_tensor"};
struct TimedLaunch {
    int kid;
    cudaEvent_t a, b;
};
static std::atomic<bool> g_timing{false};
static std::vector<TimedLaunch> g_timed;          // guarded by g_timing_mutex
static std::vector<cudaEvent_t> g_event_pool;     // guarded by g_timing_mutex
static thread_local size_t g_open = 0;            // index in g_timed of this thread's launch in flight

static cudaEvent_t take_event() {
    if (!g_event_pool.empty()) {
        cudaEvent_t e = g_event_pool.back();
        g_event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}
void launch_begin(int kid, cudaStream_t st) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (g_timing.load(std::memory_order_relaxed)) {
        std::lock_guard<std::mutex> lock(g_timing_mutex);
        TimedLaunch t{kid, take_event(), take_event()};
        cudaEventRecord(t.a, st);
        g_open = g_timed.size();
        g_timed.push_back(t);
    }
}
bool timing_active() { return g_timing.load(std::memory_order_relaxed); }
void launch_end(int kid, cudaStream_t st) {
    (void)kid;
    if (g_timing.load(std::memory_order_relaxed)) {
        std::lock_guard<std::mutex> lock(g_timing_mutex);
        if (g_open < g_timed.size()) cudaEventRecord(g_timed[g_open].b, st);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// CG table.  One block per triple, threads stride over the (2l+1)(2l2+1) band entries; Racah's sum in double with a
// log-factorial table, the same arithmetic as CGNet/cudaCG/cudaCG_sparse.cu:33-57 (the reference runs one *thread*
// per triple and leaves entries outside the band untouched; here they are written as zero).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ double lf(const double* t, int n) { return n < 2 ? 0.0 : t[n]; }

__global__ void cg_table_kernel(float* __restrict__ cg, const int* __restrict__ llls, const int64_t* __restrict__ offs,
                                int n_triples, int L1, const double* __restrict__ logfact) {
    const int k = blockIdx.x;
    if (k >= n_triples) return;
    const int code = llls[k];
    const int l = code / (L1 * L1), l1 = (code / L1) % L1, l2 = code % L1;
    const int n2 = 2 * l2 + 1, n = 2 * l + 1;
    float* out = cg + offs[k];
    const double logA0 = 0.5 * (log(2.0 * l + 1.0) + lf(logfact, l + l1 - l2) + lf(logfact, l - l1 + l2) +
                                lf(logfact, l1 + l2 - l) - lf(logfact, l1 + l2 + l + 1));
    for (int e = threadIdx.x; e < n * n2; e += blockDim.x) {
        const int m = e / n2 - l, m2 = e % n2 - l2, m1 = m - m2;
        float v = 0.f;
        if (m1 >= -l1 && m1 <= l1) {
            const int a = l2 - m1 - l, b = l1 + m2 - l, c = l1 + l2 - l, d = l1 - m1, f = l2 + m2;
            const int lo = max(0, max(a, b)), hi = min(c, min(d, f));
            const double logA = logA0 + 0.5 * (lf(logfact, l + m) + lf(logfact, l - m) + lf(logfact, l1 - m1) +
                                               lf(logfact, l1 + m1) + lf(logfact, l2 - m2) + lf(logfact, l2 + m2));
            double s = 0.0;
            for (int t = lo; t <= hi; ++t) {
                const double logB = lf(logfact, t) + lf(logfact, c - t) + lf(logfact, d - t) + lf(logfact, f - t) +
                                    lf(logfact, t - a) + lf(logfact, t - b);
                const double term = exp(logA - logB);
                s += (t & 1) ? -term : term;
            }
            v = (float)s;
        }
        out[e] = v;
    }
}

// Copy of the CG table with rows padded to a multiple of four floats; block per triple.
__global__ void cg_pad_kernel(const float* __restrict__ cg, float* __restrict__ out, const TripleRec* __restrict__ triples,
                              const int64_t* __restrict__ poff, int n_triples) {
    const int k = blockIdx.x;
    if (k >= n_triples) return;
    const TripleRec t = triples[k];
    const int n = 2 * t.l + 1, n2 = 2 * t.l2 + 1, n2p = (n2 + 3) & ~3;
    for (int e = threadIdx.x; e < n * n2p; e += blockDim.x) {
        const int r = e / n2p, c = e - r * n2p;
        out[poff[k] + e] = c < n2 ? cg[t.cgoff + r * n2 + c] : 0.f;
    }
}

static int decode_and_check(int lmax, const int32_t* llls, int n, std::vector<int>& ls, std::vector<int>& l1s,
                            std::vector<int>& l2s) {
    CGB_REQUIRE(lmax >= 0 && lmax <= kMaxLmax, "lmax out of range [0, 511]");
    CGB_REQUIRE(n >= 0 && (n == 0 || llls != nullptr), "triple list is null");
    const int L1 = lmax + 1;
    ls.resize(n);
    l1s.resize(n);
    l2s.resize(n);
    for (int k = 0; k < n; ++k) {
        const int c = llls[k];
        CGB_REQUIRE(c >= 0 && (int64_t)c < (int64_t)L1 * L1 * L1, "triple code out of range");
        const int l = c / (L1 * L1), l1 = (c / L1) % L1, l2 = c % L1;
        CGB_REQUIRE(l2 <= l1, "triples must come with l2 <= l1");
        CGB_REQUIRE(l >= l1 - l2 && l <= l1 + l2, "triple violates |l1-l2| <= l <= l1+l2");
        CGB_REQUIRE(k == 0 || l >= ls[k - 1], "triples must be grouped by non-decreasing l");
        ls[k] = l;
        l1s[k] = l1;
        l2s[k] = l2;
    }
    return CGB200_OK;
}

static int build_table(float* cg_dev, int64_t cg_len, int lmax, const int32_t* llls, int n, cudaStream_t st) {
    std::vector<int> ls, l1s, l2s;
    int rc = decode_and_check(lmax, llls, n, ls, l1s, l2s);
    if (rc) return rc;
    std::vector<int64_t> offs(n + 1, 0);
    for (int k = 0; k < n; ++k) offs[k + 1] = offs[k] + (int64_t)(2 * ls[k] + 1) * (2 * l2s[k] + 1);
    CGB_REQUIRE(cg_len == offs[n], "cg_len does not match the triple list");
    if (n == 0) return CGB200_OK;
    CGB_REQUIRE(cg_dev != nullptr, "cg_dev is null");
    const int nlf = 3 * lmax + 4;
    std::vector<double> logfact(nlf, 0.0);
    for (int i = 2; i < nlf; ++i) logfact[i] = logfact[i - 1] + log((double)i);   // cudaCG_utils.cu:83-90
    // the three temporaries are freed on every path out of this function
    struct Temps {
        double* lf = nullptr;
        int* llls = nullptr;
        int64_t* offs = nullptr;
        ~Temps() {
            cudaFree(lf);
            cudaFree(llls);
            cudaFree(offs);
        }
    } t;
    CGB_CUDA(cudaMalloc(&t.lf, nlf * sizeof(double)));
    CGB_CUDA(cudaMalloc(&t.llls, n * sizeof(int)));
    CGB_CUDA(cudaMalloc(&t.offs, (n + 1) * sizeof(int64_t)));
    CGB_CUDA(cudaMemcpyAsync(t.lf, logfact.data(), nlf * sizeof(double), cudaMemcpyHostToDevice, st));
    CGB_CUDA(cudaMemcpyAsync(t.llls, llls, n * sizeof(int), cudaMemcpyHostToDevice, st));
    CGB_CUDA(cudaMemcpyAsync(t.offs, offs.data(), (n + 1) * sizeof(int64_t), cudaMemcpyHostToDevice, st));
    launch_begin(K_CG_TABLE, st);
    cg_table_kernel<<<n, 128, 0, st>>>(cg_dev, t.llls, t.offs, n, lmax + 1, t.lf);
    launch_end(K_CG_TABLE, st);
    CGB_CUDA(cudaGetLastError());
    CGB_CUDA(cudaStreamSynchronize(st));   // one-off set-up call: the host vectors and temporaries die here
    return CGB200_OK;
}

template <typename T>
static int upload(cgb200_plan* p, const std::vector<T>& v, const T** out) {
    void* d = nullptr;
    const size_t bytes = std::max<size_t>(v.size(), 1) * sizeof(T);
    CGB_CUDA(cudaMalloc(&d, bytes));
    p->allocations.push_back(d);
    if (!v.empty()) CGB_CUDA(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    *out = (const T*)d;
    return CGB200_OK;
}

// Channel-tile edge: the largest fraction of useful lanes in the T x T register tiles, weighted by each triple's work,
// with a mild preference for 4..5 (enough arithmetic per shared-memory load, moderate register use).
static int choose_tile(const std::vector<TripleRec>& tr, bool dw) {
    static const double pref[kMaxTile + 1] = {0, 0.55, 0.80, 0.93, 1.00, 1.00, 0.96};
    int best = 1;
    double best_score = -1;
    for (int T = 1; T <= kMaxTile; ++T) {
        double useful = 0, spent = 0;
        for (const auto& t : tr) {
            const double w = (double)(2 * t.l + 1) * (2 * t.l2 + 1);
            const double n1 = (t.tau1 + T - 1) / T, n2 = (t.tau2 + T - 1) / T;
            if (dw) {
                useful += w * t.tau1;
                spent += w * n1 * T;
            } else {
                useful += w * t.tau1 * t.tau2;
                spent += w * n1 * n2 * T * T;
            }
        }
        const double score = (spent > 0 ? useful / spent : 1.0) * pref[T];
        if (score > best_score + 1e-9) {
            best_score = score;
            best = T;
        }
    }
    return best;
}

}  // namespace cgb200

using namespace cgb200;

extern "C" {

const char* cgb200_last_error(void) { return g_last_error.c_str(); }
int cgb200_version(void) { return 100; }
int cgb200_max_lmax(void) { return kMaxLmax; }
int64_t cgb200_launch_count(int reset) {
    return reset ? g_launches.exchange(0) : g_launches.load();
}

int cgb200_kernel_count(void) { return K_COUNT; }
const char* cgb200_kernel_name(int kid) { return (kid >= 0 && kid < K_COUNT) ? kKernelNames[kid] : ""; }

void cgb200_timing_enable(int on) { g_timing.store(on != 0); }

int cgb200_timing_read(double* ms, int64_t* launches, int reset) {
    CGB_REQUIRE(ms != nullptr && launches != nullptr, "null argument");
    for (int k = 0; k < K_COUNT; ++k) {
        ms[k] = 0.0;
        launches[k] = 0;
    }
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    for (const TimedLaunch& t : g_timed) {
        CGB_CUDA(cudaEventSynchronize(t.b));
        float dt = 0.f;
        CGB_CUDA(cudaEventElapsedTime(&dt, t.a, t.b));
        ms[t.kid] += dt;
        launches[t.kid] += 1;
    }
    if (reset) {
        for (const TimedLaunch& t : g_timed) {
            g_event_pool.push_back(t.a);
            g_event_pool.push_back(t.b);
        }
        g_timed.clear();
    }
    return CGB200_OK;
}

int64_t cgb200_cg_table_length(int lmax, const int32_t* llls, int n) {
    std::vector<int> ls, l1s, l2s;
    if (decode_and_check(lmax, llls, n, ls, l1s, l2s)) return -1;
    int64_t len = 0;
    for (int k = 0; k < n; ++k) len += (int64_t)(2 * ls[k] + 1) * (2 * l2s[k] + 1);
    return len;
}

int cgb200_cg_table_build(float* cg_dev, int64_t cg_len, int lmax, const int32_t* llls, int n, void* stream) {
    return build_table(cg_dev, cg_len, lmax, llls, n, (cudaStream_t)stream);
}

int cgb200_plan_create(cgb200_plan** out, int lmax, const int32_t* tau_in, const int32_t* tau_out,
                       const int32_t* llls, int n, int flags) {
    CGB_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    CGB_REQUIRE(tau_in != nullptr, "tau_in is null");
    std::vector<int> ls, l1s, l2s;
    int rc = decode_and_check(lmax, llls, n, ls, l1s, l2s);
    if (rc) return rc;
    const bool dw = (flags & CGB200_PLAN_DEPTHWISE) != 0;
    const int L1 = lmax + 1;

    cgb200_plan* p = new cgb200_plan();
    struct Guard {
        cgb200_plan* p;
        ~Guard() { if (p) cgb200_plan_destroy(p); }
    } guard{p};
    p->flags = flags;
    CGB_CUDA(cudaGetDevice(&p->device));
    CGB_CUDA(cudaDeviceGetAttribute(&p->num_sms, cudaDevAttrMultiProcessorCount, p->device));
    p->max_n = 2 * lmax + 1;

    p->tF.assign(tau_in, tau_in + L1);
    for (int l = 0; l < L1; ++l) CGB_REQUIRE(p->tF[l] >= 0 && p->tF[l] <= 32767, "tau_in out of range [0, 32767]");
    const bool has_out = tau_out != nullptr;
    if (has_out) {
        p->tO.assign(tau_out, tau_out + L1);
        for (int l = 0; l < L1; ++l) CGB_REQUIRE(p->tO[l] >= 0, "tau_out must be non-negative");
    } else {
        p->tO.assign(L1, 0);
    }

    p->cumF.assign(L1 + 1, 0);
    for (int l = 0; l < L1; ++l) p->cumF[l + 1] = p->cumF[l] + (int64_t)p->tF[l] * (2 * l + 1);
    CGB_REQUIRE(p->cumF[L1] < (1ll << 30), "input activation too long");

    // mid-channel counts and per-triple offsets (CGNet/CG_layers.py:253-262)
    std::vector<int64_t> tff64(L1, 0);
    p->triples.resize(n);
    int64_t cgoff = 0;
    for (int k = 0; k < n; ++k) {
        TripleRec& t = p->triples[k];
        t.l = ls[k];
        t.l1 = l1s[k];
        t.l2 = l2s[k];
        t.tau1 = p->tF[t.l1];
        t.tau2 = p->tF[t.l2];
        if (dw) CGB_REQUIRE(t.tau1 == t.tau2, "depthwise product needs tau_l1 == tau_l2 for every pair");
        t.nch = dw ? t.tau1 : t.tau1 * t.tau2;
        CGB_REQUIRE(tff64[t.l] + t.nch < (1ll << 31), "too many mid channels in one degree");
        t.toff = (int)tff64[t.l];
        tff64[t.l] += t.nch;
        t.f1off = (int)p->cumF[t.l1];
        t.f2off = (int)p->cumF[t.l2];
        CGB_REQUIRE(cgoff < (1ll << 31) - (1 << 20), "CG table too long");
        t.cgoff = (int)cgoff;
        cgoff += (int64_t)(2 * t.l + 1) * (2 * t.l2 + 1);
    }
    p->tFF.resize(L1);
    p->cumT.assign(L1 + 1, 0);
    p->cumFF.assign(L1 + 1, 0);
    p->cumO.assign(L1 + 1, 0);
    p->cumW.assign(L1 + 1, 0);
    for (int l = 0; l < L1; ++l) {
        p->tFF[l] = (int)tff64[l];
        CGB_REQUIRE((int64_t)p->cumT[l] + tff64[l] < (1ll << 31), "too many mid channels");
        p->cumT[l + 1] = p->cumT[l] + p->tFF[l];
        p->cumFF[l + 1] = p->cumFF[l] + tff64[l] * (2 * l + 1);
        p->cumO[l + 1] = p->cumO[l] + (int64_t)p->tO[l] * (2 * l + 1);
        p->cumW[l + 1] = p->cumW[l] + tff64[l] * p->tO[l];
    }
    for (auto& t : p->triples) {
        t.kglob = p->cumT[t.l] + t.toff;
        t.ffoff = p->cumFF[t.l] + (int64_t)t.toff * (2 * t.l + 1);
        t.woff = p->cumW[t.l] + t.toff;
    }

    const int forced_tile = (flags >> 8) & 0xF;   // CGB200_PLAN_TILE
    CGB_REQUIRE(forced_tile <= kMaxTile, "CGB200_PLAN_TILE: tile edge out of range [1, 6]");
    const int T = forced_tile ? forced_tile : choose_tile(p->triples, dw);
    p->triple_begin.assign(L1 + 1, 0);
    p->cell_begin.assign(L1 + 1, 0);
    for (int k = 0; k < n; ++k) {
        TripleRec& t = p->triples[k];
        t.nt1 = (t.tau1 + T - 1) / T;
        t.nt2 = dw ? 1 : (t.tau2 + T - 1) / T;
        t.cell0 = (int)p->cells.size();
        for (int i1 = 0; i1 < t.nt1; ++i1)
            for (int i2 = 0; i2 < t.nt2; ++i2) {
                CellRec c;
                c.triple = k;
                c.t1_0 = (short)(i1 * T);
                c.t2_0 = (short)(dw ? i1 * T : i2 * T);
                p->cells.push_back(c);
            }
        CGB_REQUIRE(p->cells.size() < (size_t)(1u << 30), "too many work cells");
        p->triple_begin[t.l + 1] = k + 1;
        p->cell_begin[t.l + 1] = (int)p->cells.size();
    }
    for (int l = 0; l < L1; ++l) {   // degrees without triples inherit the running end
        p->triple_begin[l + 1] = std::max(p->triple_begin[l + 1], p->triple_begin[l]);
        p->cell_begin[l + 1] = std::max(p->cell_begin[l + 1], p->cell_begin[l]);
    }

    // slab layouts (tile-interleaved, see PlanDev) and the forward kernel's row order
    p->cumSF.assign(L1 + 1, 0);
    p->cumSO.assign(L1 + 1, 0);
    for (int l = 0; l < L1; ++l) {
        const int64_t a = (int64_t)p->cumSF[l] + (int64_t)((p->tF[l] + T - 1) / T) * T * (2 * l + 1);
        const int64_t b = (int64_t)p->cumSO[l] + (int64_t)((p->tO[l] + T - 1) / T) * T * (2 * l + 1);
        CGB_REQUIRE(a < (1ll << 26) && b < (1ll << 26), "activation too long for the fused kernels");
        p->cumSF[l + 1] = (int)a;
        p->cumSO[l + 1] = (int)b;
        p->max_tau_out = std::max(p->max_tau_out, p->tO[l]);
    }
    for (const CellRec& c : p->cells) {
        const TripleRec& t = p->triples[c.triple];
        CellInfo ci;
        ci.cgoff = t.cgoff;
        ci.o1 = p->cumSF[t.l1] + (c.t1_0 / T) * (2 * t.l1 + 1) * T;
        ci.o2 = p->cumSF[t.l2] + (c.t2_0 / T) * (2 * t.l2 + 1) * T;
        const int ch0 = dw ? c.t1_0 : c.t1_0 * t.tau2 + c.t2_0;
        ci.wch0 = t.toff + ch0;
        ci.kch0 = t.kglob + ch0;
        ci.tau2 = t.tau2;
        ci.l1 = (short)t.l1;
        ci.l2 = (short)t.l2;
        ci.v1 = (short)std::min(T, t.tau1 - c.t1_0);
        ci.v2 = (short)std::min(T, t.tau2 - c.t2_0);
        p->cell_info.push_back(ci);
    }
    {
        std::vector<std::pair<double, int>> rows;   // (cost, l*(2*lmax+1)+mi)
        for (int l = 0; l < L1; ++l) {
            if (p->tO[l] == 0) continue;
            for (int mi = 0; mi < 2 * l + 1; ++mi) {
                double cost = 0;
                for (int k = p->triple_begin[l]; k < p->triple_begin[l + 1]; ++k) {
                    const TripleRec& t = p->triples[k];
                    const int m = mi - l;
                    const int band = std::min(t.l2, m + t.l1) - std::max(-t.l2, m - t.l1) + 1;
                    const double cells = (double)t.nt1 * t.nt2;
                    cost += cells * (band * (dw ? 6.0 * T : 4.0 * T * T + 4.0 * T) + (dw ? T : T * T) * (4.0 * p->tO[l] + 4));
                }
                rows.push_back({cost, l * (2 * lmax + 1) + mi});
            }
        }
        std::stable_sort(rows.begin(), rows.end(), [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
        for (auto& r : rows) {
            p->fwd_rows.push_back(r.second / (2 * lmax + 1));
            p->fwd_rows.push_back(r.second % (2 * lmax + 1));
        }
    }

    // tensor-core tables: forward (tile edge 2 or 4) and weight gradient (tile edge 4 or 5)
    const bool tc_common = !dw && has_out && p->max_tau_out >= 4 && p->max_tau_out <= 64 && 2 * lmax + 1 <= 128;
    p->tc_ok = tc_common && (T == 2 || T == 4);
    p->tc_gw_ok = tc_common && (T == 4 || T == 5);
    if (p->tc_ok || p->tc_gw_ok) {
        p->tc_npad.assign(L1, 0);
        for (int l = 0; l < L1; ++l) p->tc_npad[l] = p->tO[l] > 0 ? ((2 * p->tO[l] + 15) / 16) * 16 : 0;
        if ((rc = upload(p, p->tc_npad, &p->d_tc_npad))) return rc;
    }
    if (p->tc_ok) {
        const int Kc = 2 * T * T;
        p->tc_pack_off.assign(L1 + 1, 0);
        std::vector<std::pair<int, int>> order;   // (cells, l)
        for (int l = 0; l < L1; ++l) {
            const int64_t ncell = p->cell_begin[l + 1] - p->cell_begin[l];
            p->tc_pack_off[l + 1] = p->tc_pack_off[l] + ncell * 2 * p->tc_npad[l] * Kc;
            if (p->tO[l] > 0) order.push_back({(int)ncell, l});
        }
        int ncell_max = 0;
        for (auto& o : order) {
            ncell_max = std::max(ncell_max, o.first);
            p->tc_total_cells += (int64_t)o.first * ((2 * o.second + 1 + 3) / 4);
        }
        if ((rc = upload(p, p->tc_pack_off, &p->d_tc_pack_off))) return rc;
        constexpr int kMinPartCells = 24;   // a part pays for its set-up (tensor memory, barriers, pipeline fill) and one partial output
        for (int lv = 0; lv < cgb200_plan::kTcLevels; ++lv) {
            const int target = std::max((ncell_max + (1 << lv) - 1) >> lv, std::min(kMinPartCells, std::max(ncell_max, 1)));
            p->tc_parts[lv].assign(L1, 1);
            std::vector<std::pair<int, int>> by_len;   // (cells of the longest part, l)
            for (auto& o : order) {
                const int parts = std::max(1, (o.first + target - 1) / target);
                p->tc_parts[lv][o.second] = parts;
                p->tc_max_parts[lv] = std::max(p->tc_max_parts[lv], parts);
                by_len.push_back({(o.first + parts - 1) / parts, o.second});
                p->tc_longest[lv] = std::max(p->tc_longest[lv], by_len.back().first);
            }
            std::stable_sort(by_len.begin(), by_len.end(), [](const std::pair<int, int>& a, const std::pair<int, int>& b) { return a.first > b.first; });
            for (auto& o : by_len)
                for (int part = 0; part < p->tc_parts[lv][o.second]; ++part)
                    for (int m0 = 0; m0 < 2 * o.second + 1; m0 += 4) {
                        p->tc_tiles[lv].push_back(o.second);
                        p->tc_tiles[lv].push_back(m0);
                        p->tc_tiles[lv].push_back(part);
                        p->tc_tiles[lv].push_back(p->tc_parts[lv][o.second]);
                    }
            if ((rc = upload(p, p->tc_tiles[lv], &p->d_tc_tiles[lv]))) return rc;
            if ((rc = upload(p, p->tc_parts[lv], &p->d_tc_parts[lv]))) return rc;
        }
    }
    p->gff_ok = p->tc_ok && T == 4;
    p->tiles_ok = !dw && has_out;
    if (p->tiles_ok) {
        p->gff_pack_off.assign(L1 + 1, 0);
        p->gff_off.assign(L1 + 1, 0);
        for (int l = 0; l < L1; ++l) {
            const int64_t ncell = p->cell_begin[l + 1] - p->cell_begin[l];
            const int Kb = (2 * p->tO[l] + 7) & ~7;
            p->gff_pack_off[l + 1] = p->gff_pack_off[l] + (p->gff_ok ? ncell * 64 * Kb : 0);
            p->gff_off[l + 1] = p->gff_off[l] + (p->tO[l] > 0 ? ncell * (2 * l + 1) * T * T : 0);
        }
        if ((rc = upload(p, p->gff_pack_off, &p->d_gff_pack_off))) return rc;
        if ((rc = upload(p, p->gff_off, &p->d_gff_off))) return rc;
    }
    if (p->tc_gw_ok) {   // weight gradient: blocks of 128 / (2 T^2) cells, degrees with the longest contraction (2l+1) first
        const int per_block = 128 / (2 * T * T);
        for (int l = L1 - 1; l >= 0; --l) {
            if (p->tO[l] == 0) continue;
            const int ncell = p->cell_begin[l + 1] - p->cell_begin[l];
            for (int c0 = 0; c0 < ncell; c0 += per_block) {
                p->tc_gw_tiles.push_back(l);
                p->tc_gw_tiles.push_back(c0);
            }
        }
        if ((rc = upload(p, p->tc_gw_tiles, &p->d_tc_gw_tiles))) return rc;
    }

    // which triples use fragment l as first / second operand (for the gather-style input gradient)
    std::vector<int> r1b(L1 + 1, 0), r2b(L1 + 1, 0), r1l, r2l;
    for (int l = 0; l < L1; ++l) {
        for (int k = 0; k < n; ++k) {
            if (p->triples[k].l1 == l) r1l.push_back(k);
            if (p->triples[k].l2 == l) r2l.push_back(k);
        }
        r1b[l + 1] = (int)r1l.size();
        r2b[l + 1] = (int)r2l.size();
    }

    PlanDev& d = p->d;
    d.lmax = lmax;
    d.tile = T;
    d.depthwise = dw ? 1 : 0;
    d.n_triples = n;
    d.n_cells = (int)p->cells.size();
    d.has_out = has_out ? 1 : 0;
    d.n_F = p->cumF[L1];
    d.n_FF = p->cumFF[L1];
    d.n_O = p->cumO[L1];
    d.w_len = p->cumW[L1];
    d.sum_tff = p->cumT[L1];
    if ((rc = upload(p, p->triples, &d.triples))) return rc;
    if ((rc = upload(p, p->cells, &d.cells))) return rc;
    if ((rc = upload(p, p->cell_info, &d.cell_info))) return rc;
    if ((rc = upload(p, p->cell_begin, &d.cell_begin))) return rc;
    if ((rc = upload(p, p->triple_begin, &d.triple_begin))) return rc;
    if ((rc = upload(p, p->tF, &d.tF))) return rc;
    if ((rc = upload(p, p->tO, &d.tO))) return rc;
    if ((rc = upload(p, p->tFF, &d.tFF))) return rc;
    if ((rc = upload(p, p->cumF, &d.cumF))) return rc;
    if ((rc = upload(p, p->cumFF, &d.cumFF))) return rc;
    if ((rc = upload(p, p->cumO, &d.cumO))) return rc;
    if ((rc = upload(p, p->cumW, &d.cumW))) return rc;
    if ((rc = upload(p, p->cumT, &d.cumT))) return rc;
    if ((rc = upload(p, p->cumSF, &d.cumSF))) return rc;
    if ((rc = upload(p, p->cumSO, &d.cumSO))) return rc;
    if ((rc = upload(p, p->fwd_rows, &p->d_fwd_rows))) return rc;
    d.nSF = p->cumSF[L1];
    d.nSO = p->cumSO[L1];
    if ((rc = upload(p, r1b, &d.role1_begin))) return rc;
    if ((rc = upload(p, r1l, &d.role1_list))) return rc;
    if ((rc = upload(p, r2b, &d.role2_begin))) return rc;
    if ((rc = upload(p, r2l, &d.role2_list))) return rc;

    // work items of the forward product kernel
    for (int k = 0; k < n; ++k) {
        const TripleRec& t = p->triples[k];
        const int nn = 2 * t.l + 1, n1 = 2 * t.l1 + 1, n2 = 2 * t.l2 + 1;
        const int per = std::max(1, kGenThreads / nn);
        const int ncells = t.nt1 * t.nt2;
        for (int c0 = 0; c0 < ncells; c0 += per) p->gen_items.push_back({k, t.cell0 + c0, std::min(per, ncells - c0)});
        p->gen_band_bytes = std::max(p->gen_band_bytes, (size_t)((nn * n2 * 4 + 15) & ~15));
        const size_t rows2 = dw ? (size_t)t.nt1 * T : (size_t)t.nt2 * T;
        p->gen_sample_bytes = std::max(p->gen_sample_bytes, ((size_t)t.nt1 * T * n1 + rows2 * n2) * sizeof(float2));
    }
    if ((rc = upload(p, p->gen_items, &p->d_gen_items))) return rc;

    // warp-tasks of the fused weight-gradient kernel: (t1 group, t2 tile, tau_out tile) per triple
    // rows of t1 and output channels per task, by tile edge: about 32..50 complex accumulators per lane
    static const int kGwTo[kMaxTile + 1] = {0, 8, 8, 4, 4, 5, 6};
    p->gw_i = dw ? T : gw_rows_a(T);
    p->gw_to = dw ? T : kGwTo[T];
    p->gw_begin.assign(n + 1, 0);
    for (int k = 0; k < n; ++k) {
        const TripleRec& t = p->triples[k];
        const int64_t no = (p->tO[t.l] + p->gw_to - 1) / p->gw_to;
        // t1 groups never straddle a channel tile: ceil(T / I) groups per tile
        const int64_t ni = dw ? t.nt1 : (int64_t)t.nt1 * ((T + p->gw_i - 1) / p->gw_i);
        const int64_t cnt = dw ? ni * no : ni * t.nt2 * no;
        CGB_REQUIRE(p->gw_begin[k] + cnt < (1ll << 26), "too many weight-gradient tasks");
        p->gw_begin[k + 1] = p->gw_begin[k] + (int)cnt;
        const int groups = dw ? 1 : (T + p->gw_i - 1) / p->gw_i;
        for (int q1 = 0; q1 < t.nt1; ++q1)
            for (int gi = 0; gi < groups; ++gi)
                for (int q2 = 0; q2 < (dw ? 1 : t.nt2); ++q2)
                    for (int qo = 0; qo < (int)no; ++qo)
                        p->gw_tasks.push_back({k, (short)q1, (short)(dw ? gi : gi * p->gw_i), (short)q2, (short)qo,
                                               (short)(dw ? T : std::min(p->gw_i, T - gi * p->gw_i)), 0});
        CGB_REQUIRE((int)p->gw_tasks.size() == p->gw_begin[k + 1], "internal: weight-gradient task count");
    }
    {   // the warps of the weight-gradient kernel pull tasks from a queue: most expensive first
        auto cost = [&](const GwTask& tk) {
            const TripleRec& t = p->triples[tk.triple];
            double nnz = 0;
            for (int m = -t.l; m <= t.l; ++m) nnz += std::min(t.l2, m + t.l1) - std::max(-t.l2, m - t.l1) + 1;
            return (nnz + 6.0 * (2 * t.l2 + 1)) * (2.0 + tk.ni);   // the per-row part and the part shared by the rows
        };
        std::vector<std::pair<double, int>> order;
        order.reserve(p->gw_tasks.size());
        for (size_t i = 0; i < p->gw_tasks.size(); ++i) order.push_back({cost(p->gw_tasks[i]), (int)i});
        std::stable_sort(order.begin(), order.end(), [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
        std::vector<GwTask> sorted;
        sorted.reserve(order.size());
        for (auto& o : order) sorted.push_back(p->gw_tasks[o.second]);
        p->gw_tasks.swap(sorted);
    }
    if ((rc = upload(p, p->gw_tasks, &p->d_gw_tasks))) return rc;
    // entries of the fused input-gradient kernel, per fragment
    p->gf_begin.assign(L1 + 1, 0);
    for (int l = 0; l < L1; ++l) {
        for (int k = 0; k < n; ++k) {
            const TripleRec& t = p->triples[k];
            if (t.l1 == l)
                for (int j = 0; j < (dw ? 1 : t.nt2); ++j) p->gf_entries.push_back({k, 0, (short)(j * T)});
            if (t.l2 == l)
                for (int i = 0; i < (dw ? 1 : t.nt1); ++i) p->gf_entries.push_back({k, 1, (short)(i * T)});
        }
        p->gf_begin[l + 1] = (int)p->gf_entries.size();
    }
    for (const GfEntry& en : p->gf_entries) {
        const TripleRec& t = p->triples[en.triple];
        GfInfo gi;
        const bool first = en.role == 0;
        const int lo_ = first ? t.l2 : t.l1;
        gi.cgoff = t.cgoff;
        gi.go_off = p->cumSO[t.l];
        gi.fo_off = p->cumSF[lo_] + (dw ? 0 : (en.in0 / T) * (2 * lo_ + 1) * T);
        gi.kglob = t.kglob;
        gi.tau2 = t.tau2;
        gi.tff = p->tFF[t.l];
        gi.to_n = p->tO[t.l];
        gi.tau_o = first ? t.tau2 : t.tau1;
        gi.l = (short)t.l;
        gi.l1 = (short)t.l1;
        gi.l2 = (short)t.l2;
        gi.role = en.role;
        gi.in0 = en.in0;
        gi.pad_ = 0;
        gi.cell0 = t.cell0;
        gi.pad2_ = 0;
        gi.woff = t.woff;
        p->gf_info.push_back(gi);
    }
    if ((rc = upload(p, p->gf_info, &p->d_gf_info))) return rc;
    {
        // Phase 2 of the input-gradient kernel: the rows of the owned fragment, each one unit or (split) one unit for
        // the first ceil(T/2) owned channels and one for the rest, dealt to the block's warps by longest processing time
        // first.  A unit's cost is its share of the row's band length summed over the fragment's entries plus a fixed
        // part.  Two tables, [split][2 l^2 + unit].
        constexpr int kWarps = kGfWarps;
        const int ah = (T + 1) / 2, al = T - ah;
        p->gf_owner.assign((size_t)2 * 2 * L1 * L1, 255);
        for (int cfg = 0; cfg < 2; ++cfg)
        for (int l = 0; l < L1; ++l) {
            const bool split = cfg == 1 && al > 0;
            const int nt = 2 * l + 1;
            std::vector<double> row(nt, 0.0);
            for (int e = p->gf_begin[l]; e < p->gf_begin[l + 1]; ++e) {
                const TripleRec& t = p->triples[p->gf_entries[e].triple];
                const int lo_ = p->gf_entries[e].role == 0 ? t.l2 : t.l1;
                for (int r = 0; r < nt; ++r) {
                    const int mt = r - l;
                    const int len = std::min(t.l, mt + lo_) - std::max(-t.l, mt - lo_) + 1;
                    row[r] += std::max(len, 0) + 1.0;
                }
            }
            std::vector<std::pair<double, int>> units;
            for (int r = 0; r < nt; ++r) {
                units.push_back({row[r] * (0.15 + (split ? ah : T)), r});
                if (split) units.push_back({row[r] * (0.15 + al), nt + r});
            }
            std::stable_sort(units.begin(), units.end(), [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
            double load[kWarps] = {0.0};
            for (auto& u : units) {
                int best = 0;
                for (int w = 1; w < kWarps; ++w)
                    if (load[w] < load[best]) best = w;
                load[best] += u.first;
                p->gf_owner[(size_t)cfg * 2 * L1 * L1 + (size_t)2 * l * l + u.second] = (unsigned char)best;
            }
        }
        if ((rc = upload(p, p->gf_owner, &p->d_gf_owner))) return rc;
    }
    {
        // cost of a fragment's entry list ~ sum over entries of (2l+1)*tau_out*T^2 (gFF tile) + band*T^2 (contraction)
        std::vector<double> cost(L1, 0.0);
        double cmax = 0.0;
        for (int l = 0; l < L1; ++l) {
            for (int e = p->gf_begin[l]; e < p->gf_begin[l + 1]; ++e) {
                const TripleRec& t = p->triples[p->gf_entries[e].triple];
                cost[l] += (double)(2 * t.l + 1) * (p->tO[t.l] + 2.0 * (2 * t.l2 + 1)) * (dw ? T : T * T);
            }
            cmax = std::max(cmax, cost[l]);
        }
        // Order of the blocks inside a launch: longest first, by an estimate of a block's time on its critical warp
        // (the hardware hands blocks to the SMs in index order, so what is listed last forms the tail).  Per entry:
        // phase 1 in rounds of 16 warps (a load round trip per output tile plus the multiply-adds of a unit), phase 2
        // as the busiest warp's band steps (rows are dealt to 16 warps, so a fragment with few rows still walks whole
        // bands), a hand-over cost, and per block set-up and write-out.  Measured at lmax 10 with 5 and 8 channels the
        // blocks of the low degrees take 1.3-1.5 times as long as those of the high degrees, which the cost above
        // (multiply-adds, used to deal the parts) does not see.
        std::vector<double> crit(L1, 0.0);
        {
            const int NHh = dw ? T : T * T;
            const bool halves = NHh >= 4;
            for (int l = 0; l < L1; ++l) {
                const int nt = 2 * l + 1;
                for (int e = p->gf_begin[l]; e < p->gf_begin[l + 1]; ++e) {
                    const TripleRec& t = p->triples[p->gf_entries[e].triple];
                    const int lo_ = p->gf_entries[e].role == 0 ? t.l2 : t.l1;
                    const int nn = 2 * t.l + 1, to_n = p->tO[t.l];
                    const int units1 = halves ? 2 * nn : nn, kn = halves ? NHh / 2 : NHh;
                    const double c1 = (double)((units1 + kGfWarps - 1) / kGfWarps) * (90.0 * ((to_n + T - 1) / T) + (double)to_n * kn);
                    int longest = 0, sum = 0;
                    for (int r = 0; r < nt; ++r) {
                        const int mt = r - l;
                        const int len = std::max(std::min(t.l, mt + lo_) - std::max(-t.l, mt - lo_) + 1, 0);
                        longest = std::max(longest, len);
                        sum += len;
                    }
                    const double c2 = 2.0 * NHh * std::max(longest, (sum + kGfWarps - 1) / kGfWarps);
                    crit[l] += 60.0 + c1 + c2;
                }
            }
        }
        for (int lv = 0; lv < cgb200_plan::kGfLevels; ++lv) {
            const int sfac = 1 << lv;
            p->gf2_parts[lv].assign(L1, 1);
            std::vector<std::pair<double, std::array<int, 4>>> listed;
            for (int l = L1 - 1; l >= 0; --l) {   // high degrees first: they are the expensive ones
                const int n_entries = p->gf_begin[l + 1] - p->gf_begin[l];
                int parts = cmax > 0 ? (int)(sfac * cost[l] / cmax + 0.5) : 1;
                parts = std::max(1, std::min(parts, std::max(n_entries, 1)));
                p->gf2_parts[lv][l] = parts;
                p->gf2_max_parts[lv] = std::max(p->gf2_max_parts[lv], parts);
                p->gf2_longest[lv] = std::max(p->gf2_longest[lv], cost[l] / parts);
                const int ntile = (p->tF[l] + T - 1) / T;
                if (lv == 0) p->gf_total_cost += cost[l] * ntile;
                for (int q = 0; q < ntile; ++q)
                    for (int part = 0; part < parts; ++part) listed.push_back({crit[l] / parts + 300.0, {l, q, part, parts}});
            }
            std::stable_sort(listed.begin(), listed.end(),
                             [](const std::pair<double, std::array<int, 4>>& a, const std::pair<double, std::array<int, 4>>& b) { return a.first > b.first; });
            for (const auto& b : listed)
                for (int k = 0; k < 4; ++k) p->gf2_blocks[lv].push_back(b.second[k]);
            if ((rc = upload(p, p->gf2_blocks[lv], &p->d_gf2_blocks[lv]))) return rc;
            if ((rc = upload(p, p->gf2_parts[lv], &p->d_gf2_parts[lv]))) return rc;
        }
    }
    if ((rc = upload(p, p->gf_begin, &p->d_gf_begin))) return rc;

    CGB_CUDA(cudaMalloc(&p->d_status, sizeof(int)));
    p->allocations.push_back(p->d_status);
    CGB_CUDA(cudaMemset(p->d_status, 0, sizeof(int)));

    float* cg = nullptr;
    CGB_CUDA(cudaMalloc(&cg, std::max<int64_t>(cgoff, 1) * sizeof(float)));
    p->allocations.push_back(cg);
    if ((rc = build_table(cg, cgoff, lmax, llls, n, nullptr))) return rc;
    d.cg = cg;
    p->cg_len = cgoff;
    if (p->tc_ok && n > 0) {   // padded copy for the staged tensor-core forward
        std::vector<int64_t> poff(n + 1, 0);
        for (int k = 0; k < n; ++k) {
            const TripleRec& t = p->triples[k];
            poff[k + 1] = poff[k] + (int64_t)(2 * t.l + 1) * ((2 * t.l2 + 1 + 3) & ~3);
        }
        CGB_REQUIRE(poff[n] < (1ll << 31), "CG table too long");
        for (const CellRec& c : p->cells) p->cell_cgpad.push_back((int)poff[c.triple]);
        if ((rc = upload(p, p->cell_cgpad, &p->d_cell_cgpad))) return rc;
        const int64_t* d_poff = nullptr;
        if ((rc = upload(p, poff, &d_poff))) return rc;
        float* pad = nullptr;
        CGB_CUDA(cudaMalloc(&pad, poff[n] * sizeof(float)));
        p->allocations.push_back(pad);
        cg_pad_kernel<<<n, 128>>>(cg, pad, d.triples, d_poff, n);
        CGB_CUDA(cudaGetLastError());
        CGB_CUDA(cudaDeviceSynchronize());
        p->d_cg_pad = pad;
    }

    guard.p = nullptr;
    *out = p;
    return CGB200_OK;
}

void cgb200_plan_destroy(cgb200_plan* p) {
    if (!p) return;
    for (void* a : p->allocations) cudaFree(a);
    if (p->side_stream) cudaStreamDestroy(p->side_stream);
    if (p->ev_fork) cudaEventDestroy(p->ev_fork);
    if (p->ev_join) cudaEventDestroy(p->ev_join);
    delete p;
}

int cgb200_plan_query(const cgb200_plan* p, int what, int64_t* v) {
    CGB_REQUIRE(p != nullptr && v != nullptr, "null argument");
    switch (what) {
        case CGB200_Q_N_F: *v = p->d.n_F; break;
        case CGB200_Q_N_FF: *v = p->d.n_FF; break;
        case CGB200_Q_N_O: *v = p->d.n_O; break;
        case CGB200_Q_W_LEN: *v = p->d.w_len; break;
        case CGB200_Q_SUM_TFF: *v = p->d.sum_tff; break;
        case CGB200_Q_CG_LEN: *v = p->cg_len; break;
        case CGB200_Q_N_TRIPLES: *v = p->d.n_triples; break;
        case CGB200_Q_TILE: *v = p->d.tile; break;
        default: set_error("unknown query"); return CGB200_ERR_ARGUMENT;
    }
    return CGB200_OK;
}

int cgb200_plan_set_option(cgb200_plan* p, int option, int value) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    CGB_REQUIRE(option >= 0 && option < CGB200_OPT_COUNT, "unknown option");
    if (value != CGB200_AUTO) {
        switch (option) {
            case CGB200_OPT_TC_STAGES: CGB_REQUIRE(value >= 2, "CGB200_OPT_TC_STAGES must be at least 2"); break;
            case CGB200_OPT_TC_ABUF: CGB_REQUIRE(value >= 2, "CGB200_OPT_TC_ABUF must be at least 2"); break;
            case CGB200_OPT_TC_STAGED: CGB_REQUIRE(value >= 0 && value <= 2, "CGB200_OPT_TC_STAGED must be CGB200_AUTO, 0, 1 or 2"); break;
            case CGB200_OPT_TC_FWD_SPLIT:
                CGB_REQUIRE(value >= 0 && value < cgb200_plan::kTcLevels, "CGB200_OPT_TC_FWD_SPLIT must be CGB200_AUTO or 0..6");
                break;
            case CGB200_OPT_WAIT_POLLS: CGB_REQUIRE(value >= 1, "CGB200_OPT_WAIT_POLLS must be positive"); break;
            case CGB200_OPT_GRAD_MID_GEMM: CGB_REQUIRE(value >= 0 && value <= 3, "CGB200_OPT_GRAD_MID_GEMM must be CGB200_AUTO or 0..3"); break;
            default: CGB_REQUIRE(value == 0 || value == 1, "option value must be CGB200_AUTO, 0 or 1"); break;
        }
        const bool needs_tables = value == 1 || (option == CGB200_OPT_GRAD_MID_GEMM && value >= 1);
        bool have = true;
        if (option == CGB200_OPT_TC_FWD) have = p->tc_ok;
        if (option == CGB200_OPT_TC_GRAD_W) have = p->tc_gw_ok && !p->tc_gw_tiles.empty();
        if (option == CGB200_OPT_TC_GRAD_F) have = p->tc_ok && p->d.tile == 4 && p->max_n <= 64;
        if (option == CGB200_OPT_GRAD_MID_GEMM) have = p->gff_ok;
        if (option == CGB200_OPT_FWD_KEEP_MID) have = p->tiles_ok;
        if (needs_tables && !have) {
            set_error("this plan has no tables for the requested tensor-core variant (tile edge, depthwise product or channel counts)");
            return CGB200_ERR_UNSUPPORTED;
        }
    }
    p->opt[option] = value;
    return CGB200_OK;
}

int cgb200_plan_get_option(const cgb200_plan* p, int option, int* value) {
    CGB_REQUIRE(p != nullptr && value != nullptr, "null argument");
    CGB_REQUIRE(option >= 0 && option < CGB200_OPT_COUNT, "unknown option");
    *value = p->opt[option];
    return CGB200_OK;
}

int cgb200_plan_status(const cgb200_plan* p, int32_t* out) {
    CGB_REQUIRE(p != nullptr && out != nullptr, "null argument");
    int v = 0;
    CGB_CUDA(cudaMemcpy(&v, p->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) CGB_CUDA(cudaMemset(p->d_status, 0, sizeof(int)));
    *out = v;
    return CGB200_OK;
}

int cgb200_plan_t_ff(const cgb200_plan* p, int32_t* out) {
    CGB_REQUIRE(p != nullptr && out != nullptr, "null argument");
    for (size_t l = 0; l < p->tFF.size(); ++l) out[l] = p->tFF[l];
    return CGB200_OK;
}

const float* cgb200_plan_cg_table(const cgb200_plan* p) { return p ? p->d.cg : nullptr; }

}  // extern "C"
