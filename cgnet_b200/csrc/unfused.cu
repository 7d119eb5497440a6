// The two halves of the layer as separate passes over a materialised mid activation FF:
//   cgb200_cg_product_fwd / _bwd   (the reference's sparse_forward / sparse_backward)
//   cgb200_fn_wmm_fwd / _bwd       (the reference's FN_WMM_forward / FN_WMM_backward)
// They back the stand-alone modules CG_woFilter_cuda and MyBatchNormWeightMM_cuda.  The forward product is bound by
// the HBM write of FF; it stages operands and the CG band in shared memory and computes T x T channel tiles per
// thread.  The remaining kernels here are plain gather kernels (one thread per output element, deterministic sums).
#include <algorithm>

#include "common.cuh"

namespace cgb200 {

// ---------------------------------------------------------------------------------------------------------------
// CG product forward.  grid = (items, batch chunks).  A block owns `ncell` channel tiles of one triple and walks its
// batch chunk `bt` samples at a time; thread <-> (sample in group, cell, m).
// ---------------------------------------------------------------------------------------------------------------
template <int T, bool DW>
__global__ void __launch_bounds__(kGenThreads)
cg_fwd_kernel(PlanDev P, const GenItem* __restrict__ items, const float2* __restrict__ F, float2* __restrict__ FF, int B,
              int bt, int bchunk) {
    constexpr int NV = TileShape<T, DW>::NV;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const GenItem it = items[blockIdx.x];
    const TripleRec tr = P.triples[it.triple];
    const int n = 2 * tr.l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int rows1 = tr.nt1 * T, rows2 = DW ? rows1 : tr.nt2 * T;
    const int S1 = rows1 * n1, S2 = rows2 * n2, SS = S1 + S2;
    const int nband = n * n2;
    float* sC = reinterpret_cast<float*>(smem_raw);
    float2* sF = reinterpret_cast<float2*>(smem_raw + ((nband * 4 + 15) & ~15));
    const int tid = threadIdx.x;
    for (int i = tid; i < nband; i += blockDim.x) sC[i] = P.cg[tr.cgoff + i];

    const int per = it.ncell * n;
    bt = min(bt, kGenThreads / per);   // samples this item can serve per step: one thread per (sample, cell, m)
    const int bi = tid / per, rem = tid - bi * per;
    const int cj = rem / n, mi = rem - cj * n;
    const bool lane_ok = bi < bt;
    CellRec cell = P.cells[it.cell0 + (lane_ok ? cj : 0)];
    const int live1 = tr.tau1 * n1, live2 = tr.tau2 * n2;

    const int b_begin = blockIdx.y * bchunk, b_end = min(B, b_begin + bchunk);
    for (int b0 = b_begin; b0 < b_end; b0 += bt) {
        const int nb = min(bt, b_end - b0);
        __syncthreads();
        for (int i = tid; i < nb * SS; i += blockDim.x) {
            const int s = i / SS, r = i - s * SS;
            const float2* src = F + (int64_t)(b0 + s) * P.n_F;
            float2 v = make_float2(0.f, 0.f);
            if (r < S1) {
                if (r < live1) v = src[tr.f1off + r];
            } else if (r - S1 < live2) {
                v = src[tr.f2off + r - S1];
            }
            sF[i] = v;
        }
        __syncthreads();
        if (lane_ok && bi < nb) {
            float2 v[NV];
            const float2* f = sF + bi * SS;
            gen_tile<T, DW>(v, sC + mi * n2, f + cell.t1_0 * n1, n1, f + S1 + cell.t2_0 * n2, n2, mi - tr.l, tr.l1, tr.l2);
            float2* out = FF + (int64_t)(b0 + bi) * P.n_FF + tr.ffoff + mi;
#pragma unroll
            for (int idx = 0; idx < NV; ++idx)
                if (tile_valid<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau1, tr.tau2))
                    out[(int64_t)tile_channel<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau2) * n] = v[idx];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// CG product backward, gather form: one thread per element of gF, summing over every triple in which the element's
// fragment is the first operand and every triple in which it is the second (both when l1 == l2), exactly the sums of
// CGNet/cudaCG/cudaCG_sparse.cu:231-289 but driven by per-fragment triple lists built with the plan instead of a
// scan of the whole triple list per thread.
// ---------------------------------------------------------------------------------------------------------------
template <bool DW>
__global__ void __launch_bounds__(256)
cg_bwd_gather_kernel(PlanDev P, const float2* __restrict__ F, const float2* __restrict__ gFF, float2* __restrict__ gF,
                     int B) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= P.n_F) return;
    const int lt = find_degree(P.cumF, P.lmax + 1, e);
    const int nt = 2 * lt + 1;
    const int r = (int)(e - P.cumF[lt]);
    const int t = r / nt, mt = r - t * nt;   // mt = m + lt
    for (int b = blockIdx.y; b < B; b += gridDim.y) {
        const float2* Fb = F + (int64_t)b * P.n_F;
        const float2* Gb = gFF + (int64_t)b * P.n_FF;
        float2 acc = make_float2(0.f, 0.f);
        // element is F1[t][m1 = mt - lt]
        for (int q = P.role1_begin[lt]; q < P.role1_begin[lt + 1]; ++q) {
            const TripleRec tr = P.triples[P.role1_list[q]];
            const int n = 2 * tr.l + 1, n2 = 2 * tr.l2 + 1;
            const float* C = P.cg + tr.cgoff;
            const float2* F2 = Fb + tr.f2off;
            const float2* G = Gb + tr.ffoff;
            // m + l = (mt - lt) + (m2i - l2) + l must fall inside [0, n): only that range of m2 is visited
            const int shift = (mt - lt) - tr.l2 + tr.l;
            for (int m2i = max(0, -shift); m2i < min(n2, n - shift); ++m2i) {
                const int mi = shift + m2i;   // m + l
                const float c = C[mi * n2 + m2i];
                if (DW) {
                    float2 f2 = F2[t * n2 + m2i];
                    f2.x *= c;
                    f2.y *= c;
                    cfma_conj(acc, f2, G[(int64_t)t * n + mi]);
                } else {
                    for (int t2 = 0; t2 < tr.tau2; ++t2) {
                        float2 f2 = F2[t2 * n2 + m2i];
                        f2.x *= c;
                        f2.y *= c;
                        cfma_conj(acc, f2, G[(int64_t)(t * tr.tau2 + t2) * n + mi]);
                    }
                }
            }
        }
        // element is F2[t][m2 = mt - lt]
        for (int q = P.role2_begin[lt]; q < P.role2_begin[lt + 1]; ++q) {
            const TripleRec tr = P.triples[P.role2_list[q]];
            const int n = 2 * tr.l + 1, n1 = 2 * tr.l1 + 1, n2 = nt;
            const float* C = P.cg + tr.cgoff;
            const float2* F1 = Fb + tr.f1off;
            const float2* G = Gb + tr.ffoff;
            const int shift = (mt - lt) - tr.l1 + tr.l;
            for (int m1i = max(0, -shift); m1i < min(n1, n - shift); ++m1i) {
                const int mi = shift + m1i;
                const float c = C[mi * n2 + mt];
                if (DW) {
                    float2 f1 = F1[t * n1 + m1i];
                    f1.x *= c;
                    f1.y *= c;
                    cfma_conj(acc, f1, G[(int64_t)t * n + mi]);
                } else {
                    for (int t1 = 0; t1 < tr.tau1; ++t1) {
                        float2 f1 = F1[t1 * n1 + m1i];
                        f1.x *= c;
                        f1.y *= c;
                        cfma_conj(acc, f1, G[(int64_t)(t1 * tr.tau2 + t) * n + mi]);
                    }
                }
            }
        }
        gF[(int64_t)b * P.n_F + e] = acc;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Fragment-norm statistics from a materialised FF (CGNet/cudaCG/cudaCG_FNWMM.cu:29-79): per mid channel k of degree l
// sigma = sqrt(E|z|^2 - (E|z|)^2) over (b, m) with double accumulation, then the moving average in fp32 storage.
// grid = (channel chunks, degrees); a block owns kc channels; thread <-> (batch slot, channel, m); fixed-order tree.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kStatThreads = 256;

__device__ __forceinline__ float moving_std(float old, double sigma, float cnt) {
    float s = old * (cnt / (cnt + 1.f));              // FNWMM.cu:75
    return (float)((double)s + sigma / (double)(cnt + 1.f));   // FNWMM.cu:76
}

__global__ void __launch_bounds__(kStatThreads)
fn_stats_kernel(PlanDev P, const float2* __restrict__ FF, float* __restrict__ stds, float cnt, int B) {
    __shared__ double s1[kStatThreads], s2[kStatThreads];
    const int l = blockIdx.y;
    const int n = 2 * l + 1;
    const int KC = max(1, kStatThreads / n);
    const int k0 = blockIdx.x * KC;
    const int tff = P.tFF[l];
    if (k0 >= tff) return;
    const int kc = min(KC, tff - k0);
    const int J = kc * n;                  // contiguous complex elements of this chunk inside one sample
    const int nslots = kStatThreads / J;   // >= 1 because KC*n <= kStatThreads (n <= kStatThreads is checked on the host)
    const int tid = threadIdx.x;
    const int slot = tid / J, j = tid - slot * J;
    double a1 = 0.0, a2 = 0.0;
    if (slot < nslots) {
        const float2* src = FF + P.cumFF[l] + (int64_t)k0 * n + j;
        for (int b = slot; b < B; b += nslots) {
            const float2 z = src[(int64_t)b * P.n_FF];
            const float nrm = z.x * z.x + z.y * z.y;
            a2 += (double)nrm;
            a1 += sqrt((double)nrm);
        }
    }
    s1[tid] = a1;
    s2[tid] = a2;
    __syncthreads();
    if (tid < kc) {
        double m1 = 0.0, m2 = 0.0;
        for (int s = 0; s < nslots; ++s)
            for (int m = 0; m < n; ++m) {
                m1 += s1[s * J + tid * n + m];
                m2 += s2[s * J + tid * n + m];
            }
        const double N = (double)B * n;
        double var = m2 / N - (m1 / N) * (m1 / N);
        const double sigma = var > 0.0 ? sqrt(var) : 0.0;
        const int k = P.cumT[l] + k0 + tid;
        stds[k] = moving_std(stds[k], sigma, cnt);
    }
}

// Mixing forward  O_l[b] = W_l diag(1/sigma) FF_l[b]  (CGNet/cudaCG/cudaCG_FNWMM.cu:81-123, which runs one thread per
// output element and so reads every FF element tau_out times).  Here a block owns (degree l, sample b) and reads
// FF_l[b], a contiguous (t_FF x (2l+1)) matrix, exactly once with coalesced loads: thread <-> (row slot kk, column m),
// walking the rows kk, kk + KC, ...; it keeps the partial sums of up to kWmmTo output channels for its column in
// registers (the weights W[to][k] / sigma_k of a row are the same for the threads of a row slot: broadcast loads), and
// the row slots are added in slot order through shared memory, so the sum has a fixed order.
constexpr int kWmmTo = 16;
__global__ void __launch_bounds__(kStatThreads)
wmm_fwd_kernel(PlanDev P, const float2* __restrict__ FF, const float2* __restrict__ W, const float* __restrict__ stds,
               float eps, float2* __restrict__ O, int B) {
    __shared__ float2 red[kStatThreads];
    const int l = blockIdx.y;
    const int n = 2 * l + 1;
    const int tff = P.tFF[l], to_n = P.tO[l];
    if (to_n == 0) return;
    const int KC = max(1, kStatThreads / n);   // row slots: KC * n <= kStatThreads (n <= kStatThreads is checked on the host)
    const int tid = threadIdx.x;
    const int kk = tid / n, mi = tid - kk * n;
    const bool live = kk < KC;
    const float2* Wl = W + P.cumW[l];
    const float* sd = stds ? stds + P.cumT[l] : nullptr;
    for (int b = blockIdx.x; b < B; b += gridDim.x) {
        const float2* src = FF + (int64_t)b * P.n_FF + P.cumFF[l] + mi;
        float2* dst = O + (int64_t)b * P.n_O + P.cumO[l] + mi;
        for (int to0 = 0; to0 < to_n; to0 += kWmmTo) {
            float2 acc[kWmmTo];
#pragma unroll
            for (int i = 0; i < kWmmTo; ++i) acc[i] = make_float2(0.f, 0.f);
            if (live) {
                for (int k = kk; k < tff; k += KC) {
                    float2 z = src[(int64_t)k * n];
                    if (sd) {
                        const float inv = 1.f / fmaxf(eps, sd[k]);
                        z.x *= inv;
                        z.y *= inv;
                    }
#pragma unroll
                    for (int i = 0; i < kWmmTo; ++i)
                        if (to0 + i < to_n) cfma(acc[i], Wl[(int64_t)(to0 + i) * tff + k], z);
                }
            }
#pragma unroll
            for (int i = 0; i < kWmmTo; ++i) {
                if (to0 + i >= to_n) break;
                __syncthreads();
                red[tid] = acc[i];
                __syncthreads();
                if (tid < n) {
                    float2 sum = make_float2(0.f, 0.f);
                    for (int q = 0; q < KC; ++q) {
                        const float2 v = red[q * n + tid];
                        sum.x += v.x;
                        sum.y += v.y;
                    }
                    dst[(int64_t)(to0 + i) * n - mi + tid] = sum;
                }
            }
        }
    }
}

// gFF = diag(1/sigma) W^H gO, one thread per element (CGNet/cudaCG/cudaCG_FNWMM.cu:169-211).
__global__ void __launch_bounds__(256)
wmm_bwd_mid_kernel(PlanDev P, const float2* __restrict__ gO, const float2* __restrict__ W, const float* __restrict__ stds,
                   float eps, float2* __restrict__ gFF, int B) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= P.n_FF) return;
    const int l = find_degree(P.cumFF, P.lmax + 1, e);
    const int n = 2 * l + 1;
    const int64_t r = e - P.cumFF[l];
    const int k = (int)(r / n), mi = (int)(r - (int64_t)k * n);
    const int tff = P.tFF[l], to_n = P.tO[l];
    const float inv = stds ? 1.f / fmaxf(eps, stds[P.cumT[l] + k]) : 1.f;
    const float2* Wcol = W + P.cumW[l] + k;
    for (int b = blockIdx.y; b < B; b += gridDim.y) {
        const float2* g = gO + (int64_t)b * P.n_O + P.cumO[l] + mi;
        float2 acc = make_float2(0.f, 0.f);
        for (int to = 0; to < to_n; ++to) cfma_conj(acc, Wcol[(int64_t)to * tff], g[to * n]);
        acc.x *= inv;
        acc.y *= inv;
        gFF[(int64_t)b * P.n_FF + e] = acc;
    }
}

// gW[to][k] = (1/sigma_k) sum_{b,m} conj(FF[b,k,m]) gO[b,to,m]  (CGNet/cudaCG/cudaCG_FNWMM.cu:126-167, which adds over
// the batch with atomicAdd; here the sum runs in a fixed order).  Same block decomposition as fn_stats_kernel, eight
// output channels at a time.
constexpr int kGwTo = 8;
__global__ void __launch_bounds__(kStatThreads)
wmm_bwd_w_kernel(PlanDev P, const float2* __restrict__ gO, const float2* __restrict__ FF, const float* __restrict__ stds,
                 float eps, float2* __restrict__ gW, int B) {
    __shared__ float2 red[kStatThreads];
    const int l = blockIdx.y;
    const int n = 2 * l + 1;
    const int KC = max(1, kStatThreads / n);
    const int k0 = blockIdx.x * KC;
    const int tff = P.tFF[l], to_n = P.tO[l];
    if (k0 >= tff) return;
    const int kc = min(KC, tff - k0);
    const int J = kc * n;
    const int nslots = kStatThreads / J;
    const int tid = threadIdx.x;
    const int slot = tid / J, j = tid - slot * J;
    const int mi = j % n;
    const bool live = slot < nslots;
    const float2* src = FF + P.cumFF[l] + (int64_t)k0 * n + j;
    for (int to0 = 0; to0 < to_n; to0 += kGwTo) {
        float2 acc[kGwTo];
#pragma unroll
        for (int i = 0; i < kGwTo; ++i) acc[i] = make_float2(0.f, 0.f);
        if (live) {
            for (int b = slot; b < B; b += nslots) {
                const float2 z = src[(int64_t)b * P.n_FF];
                const float2* g = gO + (int64_t)b * P.n_O + P.cumO[l] + mi;
#pragma unroll
                for (int i = 0; i < kGwTo; ++i)
                    if (to0 + i < to_n) cfma_conj(acc[i], z, g[(to0 + i) * n]);
            }
        }
#pragma unroll
        for (int i = 0; i < kGwTo; ++i) {
            if (to0 + i >= to_n) break;
            __syncthreads();
            red[tid] = acc[i];
            __syncthreads();
            if (tid < kc) {
                float2 s = make_float2(0.f, 0.f);
                for (int sl = 0; sl < nslots; ++sl)
                    for (int m = 0; m < n; ++m) {
                        const float2 v = red[sl * J + tid * n + m];
                        s.x += v.x;
                        s.y += v.y;
                    }
                const float inv = stds ? 1.f / fmaxf(eps, stds[P.cumT[l] + k0 + tid]) : 1.f;
                gW[P.cumW[l] + (int64_t)(to0 + i) * tff + k0 + tid] = make_float2(s.x * inv, s.y * inv);
            }
        }
    }
}

}  // namespace cgb200

using namespace cgb200;

namespace {

int check_common(const cgb200_plan* p, int64_t B) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    CGB_REQUIRE(B >= 0 && B < (1ll << 31), "batch size out of range");
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    CGB_REQUIRE(dev == p->device, "the plan belongs to another CUDA device than the current one");
    return CGB200_OK;
}

bool aligned8(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; }

template <int T, bool DW>
int launch_cg_fwd(const cgb200_plan* p, const GenItem* items, int n_items, const float2* F, float2* FF, int B, int bt,
                  int bchunk, int nby, size_t smem, cudaStream_t st) {
    auto kern = cg_fwd_kernel<T, DW>;
    if (smem > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_begin(K_CG_FWD, st);
    kern<<<dim3(n_items, nby), kGenThreads, smem, st>>>(p->d, items, F, FF, B, bt, bchunk);
    launch_end(K_CG_FWD, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // namespace


extern "C" {

int cgb200_cg_product_fwd(const cgb200_plan* p, const float* F, float* FF, int64_t B, void* stream) {
    int rc = check_common(p, B);
    if (rc) return rc;
    if (B == 0 || p->d.n_FF == 0) return CGB200_OK;
    CGB_REQUIRE(F != nullptr && FF != nullptr, "F or FF is null");
    CGB_REQUIRE(aligned8(F) && aligned8(FF), "F and FF must be 8-byte aligned");
    const GenItem* items = p->d_gen_items;
    const int n_items = (int)p->gen_items.size();
    const size_t band = p->gen_band_bytes, sample = p->gen_sample_bytes;
    if (n_items == 0) return CGB200_OK;
    CGB_REQUIRE(2 * p->d.lmax + 1 <= kGenThreads, "lmax too large for the product kernel (2l+1 > 256)");
    const size_t budget = 200 * 1024;
    if (band + sample > budget) {
        set_error("a single triple's operands exceed shared memory (tau*(2l+1) too large for the product kernel)");
        return CGB200_ERR_UNSUPPORTED;
    }
    // samples staged per step: enough to fill the block, bounded by a 64 KB target so several blocks share an SM
    const size_t soft = std::max(band + sample, (size_t)64 * 1024);
    int bt = (int)std::min<int64_t>(B, std::min<int64_t>(kGenThreads, (int64_t)((soft - band) / std::max<size_t>(sample, 8))));
    bt = std::max(bt, 1);
    const int steps = (int)((B + bt - 1) / bt);
    int nby = std::max(1, std::min(steps, (8 * p->num_sms + n_items - 1) / n_items));
    nby = std::min(nby, 65535);
    int bchunk = (int)((steps + nby - 1) / nby) * bt;
    nby = (int)((B + bchunk - 1) / bchunk);
    const size_t smem = band + (size_t)bt * sample;
    CGB_DISPATCH_TILE(p->d.tile, p->d.depthwise,
                      rc = (launch_cg_fwd<TT, DD>(p, items, n_items, (const float2*)F, (float2*)FF, (int)B, bt, bchunk, nby,
                                                  smem, (cudaStream_t)stream)));
    return rc;
}

int cgb200_cg_product_bwd(const cgb200_plan* p, const float* F, const float* gFF, float* gF, int64_t B, void* stream) {
    int rc = check_common(p, B);
    if (rc) return rc;
    if (B == 0 || p->d.n_F == 0) return CGB200_OK;
    CGB_REQUIRE(F != nullptr && gF != nullptr && (gFF != nullptr || p->d.n_FF == 0), "null buffer");
    CGB_REQUIRE(aligned8(F) && aligned8(gFF) && aligned8(gF), "buffers must be 8-byte aligned");
    const int gx = (int)((p->d.n_F + 255) / 256);
    const int gy = (int)std::min<int64_t>(B, 65535);
    launch_begin(K_CG_BWD, (cudaStream_t)stream);
    if (p->d.depthwise)
        cg_bwd_gather_kernel<true><<<dim3(gx, gy), 256, 0, (cudaStream_t)stream>>>(p->d, (const float2*)F, (const float2*)gFF, (float2*)gF, (int)B);
    else
        cg_bwd_gather_kernel<false><<<dim3(gx, gy), 256, 0, (cudaStream_t)stream>>>(p->d, (const float2*)F, (const float2*)gFF, (float2*)gF, (int)B);
    launch_end(K_CG_BWD, (cudaStream_t)stream);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

static int chunk_grid(const cgb200_plan* p, dim3* grid) {
    int gx = 1;
    for (int l = 0; l <= p->d.lmax; ++l) {
        const int n = 2 * l + 1;
        CGB_REQUIRE(n <= kStatThreads, "lmax too large for the fragment-norm kernels (2l+1 > 256)");
        const int KC = std::max(1, kStatThreads / n);
        gx = std::max(gx, (p->tFF[l] + KC - 1) / KC);
    }
    *grid = dim3(gx, p->d.lmax + 1);
    return CGB200_OK;
}

int cgb200_fn_wmm_fwd(const cgb200_plan* p, const float* FF, const float* W, float* stds, float cnt, float eps,
                      int flags, float* O, int64_t B, void* stream) {
    int rc = check_common(p, B);
    if (rc) return rc;
    CGB_REQUIRE(p->d.has_out, "the plan was created without tau_out");
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    if (B == 0 || p->d.n_O == 0) return CGB200_OK;
    CGB_REQUIRE(O != nullptr && (FF != nullptr || p->d.n_FF == 0) && (W != nullptr || p->d.w_len == 0), "null buffer");
    CGB_REQUIRE(aligned8(FF) && aligned8(W) && aligned8(O), "buffers must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (fn && (flags & CGB200_FN_UPDATE) && p->d.sum_tff > 0) {
        dim3 grid;
        if ((rc = chunk_grid(p, &grid))) return rc;
        launch_begin(K_FN_STATS, st);
        fn_stats_kernel<<<grid, kStatThreads, 0, st>>>(p->d, (const float2*)FF, stds, cnt, (int)B);
        launch_end(K_FN_STATS, st);
        CGB_CUDA(cudaGetLastError());
    }
    {
        dim3 chk;
        if ((rc = chunk_grid(p, &chk))) return rc;   // 2 lmax + 1 <= block size
    }
    const int gx = (int)std::min<int64_t>(B, 65535);
    launch_begin(K_WMM_FWD, st);
    wmm_fwd_kernel<<<dim3(gx, p->d.lmax + 1), kStatThreads, 0, st>>>(p->d, (const float2*)FF, (const float2*)W, fn ? stds : nullptr, eps,
                                                                      (float2*)O, (int)B);
    launch_end(K_WMM_FWD, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

int cgb200_fn_wmm_bwd(const cgb200_plan* p, const float* gO, const float* FF, const float* W, const float* stds,
                      float eps, int flags, float* gFF, float* gW, int64_t B, void* stream) {
    int rc = check_common(p, B);
    if (rc) return rc;
    CGB_REQUIRE(p->d.has_out, "the plan was created without tau_out");
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    CGB_REQUIRE(aligned8(gO) && aligned8(FF) && aligned8(W) && aligned8(gFF) && aligned8(gW), "buffers must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (p->d.w_len > 0) {
        CGB_REQUIRE(gW != nullptr, "gW is null");
        if (B == 0) {
            CGB_CUDA(cudaMemsetAsync(gW, 0, p->d.w_len * sizeof(float2), st));
        } else {
            CGB_REQUIRE(gO != nullptr && FF != nullptr, "null buffer");
            dim3 grid;
            if ((rc = chunk_grid(p, &grid))) return rc;
            launch_begin(K_WMM_BWD_W, st);
            wmm_bwd_w_kernel<<<grid, kStatThreads, 0, st>>>(p->d, (const float2*)gO, (const float2*)FF, fn ? stds : nullptr, eps, (float2*)gW, (int)B);
            launch_end(K_WMM_BWD_W, st);
            CGB_CUDA(cudaGetLastError());
        }
    }
    if (B > 0 && p->d.n_FF > 0) {
        CGB_REQUIRE(gFF != nullptr && gO != nullptr && W != nullptr, "null buffer");
        const int64_t gx64 = (p->d.n_FF + 255) / 256;
        CGB_REQUIRE(gx64 < (1ll << 31), "mid activation too long for one launch");
        const int gy = (int)std::min<int64_t>(B, 65535);
        launch_begin(K_WMM_BWD_MID, st);
        wmm_bwd_mid_kernel<<<dim3((unsigned)gx64, gy), 256, 0, st>>>(p->d, (const float2*)gO, (const float2*)W, fn ? stds : nullptr, eps, (float2*)gFF, (int)B);
        launch_end(K_WMM_BWD_MID, st);
        CGB_CUDA(cudaGetLastError());
    }
    return CGB200_OK;
}

}  // extern "C"
