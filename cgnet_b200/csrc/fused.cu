// The whole CG layer without a materialised mid activation: cgb200_layer_fwd / cgb200_layer_bwd.
//
// Layout idea: the activations are first transposed to sample-fastest order, Ft[element][Bp] (Bp = batch rounded up
// to 32, padded with zeros), and every warp works on one group of 32 samples, one sample per lane.  Then everything
// except the sample is uniform across a warp: the (l, l1, l2, m, m2) band loops never diverge, CG coefficients, mixing
// weights and norm factors are warp-uniform loads, operand loads are 256-byte coalesced lines that stay in L1, and the
// sums over the batch that the statistics and the weight gradient need are fixed-order warp-shuffle trees.  No float
// atomics anywhere: every output element has exactly one owner and every sum a fixed order.
//
//   prep          F (and gO) -> Ft (gOt); 1/max(eps, std) per mid channel when the statistics are not being updated
//   stats         training only: per mid channel std of |FF| over (b, m) from on-the-fly FF; moving average; 1/max(eps,.)
//   fwd           O[b, l, :, m] = sum over the cells of degree l of  W_l[:, k] * (FF[b, k, m] / std_k)
//   grad_w        gW_l[to, (t1,t2)] = (1/std) sum_{b, m2} conj(F2[t2, m2]) * sum_m C[m, m2] conj(F1[t1, m-m2]) gO[to, m]
//   grad_f        gF via gFF tiles built from gO and W in registers, contracted with conj(F) and C into per-warp
//                 shared-memory accumulators that one block owns
#include <algorithm>

#include "common.cuh"

namespace cgb200 {

constexpr int kWarp = 32;
constexpr int kFwdWarps = 8;     // warps of a forward block = slices of the degree's cell list
constexpr int kFwdTo = 16;       // output channels accumulated in registers per pass
constexpr int kGwWarps = 4;
constexpr int kGfWarpsMax = 8;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------------------------
// prep: up to two transposes src[B][N] -> dst[N][Bp] in one launch (blockIdx.z picks the job), plus the norm factors.
// ---------------------------------------------------------------------------------------------------------------
struct PrepJob {
    const float2* src;
    float2* dst;
    int64_t N;
};
__global__ void __launch_bounds__(256)
prep_kernel(PrepJob j0, PrepJob j1, int B, int Bp, const float* __restrict__ stds, float eps, float* __restrict__ inv,
            int n_inv) {
    __shared__ float2 tile[32][33];
    const PrepJob job = blockIdx.z == 0 ? j0 : j1;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    if (blockIdx.z == 0 && inv != nullptr) {   // norm factors ride along with job 0
        const int64_t stride = (int64_t)gridDim.x * gridDim.y * 256;
        for (int64_t k = ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * 256 + threadIdx.x; k < n_inv; k += stride)
            inv[k] = stds ? 1.f / fmaxf(eps, stds[k]) : 1.f;
    }
    const int g = blockIdx.y;
    for (int64_t e0 = (int64_t)blockIdx.x * 32; e0 < job.N; e0 += (int64_t)gridDim.x * 32) {
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int b = g * 32 + ty + 8 * k;
            const int64_t e = e0 + tx;
            tile[ty + 8 * k][tx] = (b < B && e < job.N) ? job.src[(int64_t)b * job.N + e] : make_float2(0.f, 0.f);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t e = e0 + ty + 8 * k;
            if (e < job.N) job.dst[e * Bp + g * 32 + tx] = tile[tx][ty + 8 * k];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// stats: one block per cell.  Warps share the (sample group, m) pairs of the cell; a lane accumulates |z| and |z|^2 of
// its own sample in fp32 over the pairs of its warp, the lanes are then summed in double by a shuffle tree and the
// warps in index order.  Same quantity as CGNet/cudaCG/cudaCG_FNWMM.cu:55-77, which takes the square root in double:
// here |z| = r + e/(2r) with r = sqrtf(|z|^2) and e = |z|^2 - r*r computed exactly by one fma, so that the variance
// E|z|^2 - (E|z|)^2 of a channel whose moduli are all equal (a single sample of degree 0, say) still comes out as 0
// instead of the ~1e-7 relative rounding of r.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float moving_std_f(float old, double sigma, float cnt) {
    const float s = old * (cnt / (cnt + 1.f));
    return (float)((double)s + sigma / (double)(cnt + 1.f));
}

template <int T, bool DW>
__global__ void __launch_bounds__(256)
fused_stats_kernel(PlanDev P, const float2* __restrict__ Ft, float* __restrict__ stds, float* __restrict__ inv, float cnt,
                   float eps, int B, int Bp) {
    constexpr int NV = TileShape<T, DW>::NV;
    __shared__ double red[8][NV][2];
    const CellRec cell = P.cells[blockIdx.x];
    const TripleRec tr = P.triples[cell.triple];
    const int n = 2 * tr.l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = Bp >> 5;
    float s1[NV], s1c[NV], s2[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) s1[i] = s1c[i] = s2[i] = 0.f;
    const float* C = P.cg + tr.cgoff;
    for (int task = warp; task < G * n; task += 8) {
        const int g = task / n, mi = task - g * n;
        const float2* f1 = Ft + ((int64_t)tr.f1off + cell.t1_0 * n1) * Bp + g * 32 + lane;
        const float2* f2 = Ft + ((int64_t)tr.f2off + cell.t2_0 * n2) * Bp + g * 32 + lane;
        float2 v[NV];
        gen_tile<T, DW>(v, C + mi * n2, f1, n1, f2, n2, mi - tr.l, tr.l1, tr.l2, Bp);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float nrm = v[i].x * v[i].x + v[i].y * v[i].y;
            const float r = sqrtf(nrm);
            s2[i] += nrm;
            s1[i] += r;
            if (nrm > 0.f) s1c[i] += __fdividef(0.5f * fmaf(-r, r, nrm), r);
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const double a = warp_sum((double)s1[i] + (double)s1c[i]), b = warp_sum((double)s2[i]);
        if (lane == 0) {
            red[warp][i][0] = a;
            red[warp][i][1] = b;
        }
    }
    __syncthreads();
    const int idx = threadIdx.x;
    if (idx < NV && tile_valid<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau1, tr.tau2)) {
        double m1 = 0.0, m2 = 0.0;
        for (int w = 0; w < 8; ++w) {
            m1 += red[w][idx][0];
            m2 += red[w][idx][1];
        }
        const double N = (double)B * n;
        const double var = m2 / N - (m1 / N) * (m1 / N);
        const double sigma = var > 0.0 ? sqrt(var) : 0.0;
        const int k = tr.kglob + tile_channel<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau2);
        const float s = moving_std_f(stds[k], sigma, cnt);
        stds[k] = s;
        inv[k] = 1.f / fmaxf(eps, s);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// forward: block = (degree l, m, sample group); its warps take the cells of the degree round-robin, each lane keeps
// up to kFwdTo output channels of its sample in registers; the warps' partial sums are added in index order.
// ---------------------------------------------------------------------------------------------------------------
template <int T, bool DW>
__global__ void __launch_bounds__(kFwdWarps * kWarp)
fused_fwd_kernel(PlanDev P, const float2* __restrict__ Ft, const float2* __restrict__ W, const float* __restrict__ inv,
                 float2* __restrict__ O, int B, int Bp) {
    constexpr int NV = TileShape<T, DW>::NV;
    __shared__ float2 red[kFwdWarps][kFwdTo][kWarp];
    // blockIdx.x enumerates (l, m): index l*l + (m + l)
    int l = (int)sqrtf((float)blockIdx.x);
    while ((l + 1) * (l + 1) <= (int)blockIdx.x) ++l;
    while (l * l > (int)blockIdx.x) --l;
    const int mi = blockIdx.x - l * l;
    const int n = 2 * l + 1;
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int to_n = P.tO[l];
    if (to_n == 0) return;
    const int tff = P.tFF[l];
    const int c_begin = P.cell_begin[l], c_end = P.cell_begin[l + 1];
    const float2* Wl = W + P.cumW[l];
    const int b = g * 32 + lane;

    for (int to0 = 0; to0 < to_n; to0 += kFwdTo) {
        float2 o[kFwdTo];
#pragma unroll
        for (int t = 0; t < kFwdTo; ++t) o[t] = make_float2(0.f, 0.f);
        for (int c = c_begin + warp; c < c_end; c += kFwdWarps) {
            const CellRec cell = P.cells[c];
            const TripleRec tr = P.triples[cell.triple];
            const int n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
            const float2* f1 = Ft + ((int64_t)tr.f1off + cell.t1_0 * n1) * Bp + g * 32 + lane;
            const float2* f2 = Ft + ((int64_t)tr.f2off + cell.t2_0 * n2) * Bp + g * 32 + lane;
            float2 v[NV];
            gen_tile<T, DW>(v, P.cg + tr.cgoff + mi * n2, f1, n1, f2, n2, mi - l, tr.l1, tr.l2, Bp);
#pragma unroll
            for (int idx = 0; idx < NV; ++idx) {
                if (!tile_valid<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau1, tr.tau2)) continue;   // warp-uniform
                const int ch = tile_channel<T, DW>(idx, cell.t1_0, cell.t2_0, tr.tau2);
                const float s = __ldg(inv + tr.kglob + ch);
                const float2 x = make_float2(v[idx].x * s, v[idx].y * s);
                const float2* w = Wl + (int64_t)to0 * tff + tr.toff + ch;
#pragma unroll
                for (int t = 0; t < kFwdTo; ++t)
                    if (to0 + t < to_n) cfma(o[t], __ldg(w + (int64_t)t * tff), x);
            }
        }
        __syncthreads();   // protects `red` from the previous pass
#pragma unroll
        for (int t = 0; t < kFwdTo; ++t) red[warp][t][lane] = o[t];
        __syncthreads();
        for (int t = warp; t < kFwdTo && to0 + t < to_n; t += kFwdWarps) {
            float2 s = red[0][t][lane];
#pragma unroll
            for (int w = 1; w < kFwdWarps; ++w) {
                s.x += red[w][t][lane].x;
                s.y += red[w][t][lane].y;
            }
            if (b < B) O[(int64_t)b * P.n_O + P.cumO[l] + (int64_t)(to0 + t) * n + mi] = s;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// weight gradient, full product.  Warp-task = (triple, I consecutive t1, one t2 tile, one tau_out tile).  A lane keeps
// acc[o][i][j] for its own sample; the sample groups are visited in order and the lanes summed at the end.
// ---------------------------------------------------------------------------------------------------------------
template <int T, int I>
__global__ void __launch_bounds__(kGwWarps * kWarp)
fused_gw_kernel(PlanDev P, const int* __restrict__ task_begin, int n_tasks, const float2* __restrict__ Ft,
                const float2* __restrict__ gOt, const float* __restrict__ inv, float2* __restrict__ gW, int Bp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int task = blockIdx.x * kGwWarps + warp;
    if (task >= n_tasks) return;
    // triple of this task: last k with task_begin[k] <= task
    int lo = 0, hi = P.n_triples;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (task_begin[mid] <= task) lo = mid; else hi = mid;
    }
    const TripleRec tr = P.triples[lo];
    const int l = tr.l, n = 2 * l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int to_n = P.tO[l], tff = P.tFF[l];
    const int no = (to_n + T - 1) / T;
    int r = task - task_begin[lo];
    const int io = r % no;
    r /= no;
    const int ij = r % tr.nt2, ii = r / tr.nt2;
    const int t1_0 = ii * I, t2_0 = ij * T, to0 = io * T;
    const float* C = P.cg + tr.cgoff;
    const int G = Bp >> 5;

    float2 acc[T][I][T];
#pragma unroll
    for (int o = 0; o < T; ++o)
#pragma unroll
        for (int i = 0; i < I; ++i)
#pragma unroll
            for (int j = 0; j < T; ++j) acc[o][i][j] = make_float2(0.f, 0.f);

    for (int g = 0; g < G; ++g) {
        const float2* f1 = Ft + ((int64_t)tr.f1off + t1_0 * n1) * Bp + g * 32 + lane;
        const float2* f2 = Ft + ((int64_t)tr.f2off + t2_0 * n2) * Bp + g * 32 + lane;
        const float2* go = gOt + (P.cumO[l] + (int64_t)to0 * n) * Bp + g * 32 + lane;
        for (int m2 = -tr.l2; m2 <= tr.l2; ++m2) {
            float2 Y[T][I];
#pragma unroll
            for (int o = 0; o < T; ++o)
#pragma unroll
                for (int i = 0; i < I; ++i) Y[o][i] = make_float2(0.f, 0.f);
            const int mlo = max(-l, m2 - tr.l1), mhi = min(l, m2 + tr.l1);
            for (int m = mlo; m <= mhi; ++m) {
                const float c = C[(m + l) * n2 + m2 + tr.l2];
                float2 a[I];
#pragma unroll
                for (int i = 0; i < I; ++i) {
                    a[i] = f1[(int64_t)(i * n1 + (m - m2) + tr.l1) * Bp];
                    a[i].x *= c;
                    a[i].y *= c;
                }
#pragma unroll
                for (int o = 0; o < T; ++o) {
                    const float2 gv = go[(int64_t)(o * n + m + l) * Bp];
#pragma unroll
                    for (int i = 0; i < I; ++i) cfma_conj(Y[o][i], a[i], gv);
                }
            }
            float2 bj[T];
#pragma unroll
            for (int j = 0; j < T; ++j) bj[j] = f2[(int64_t)(j * n2 + m2 + tr.l2) * Bp];
#pragma unroll
            for (int o = 0; o < T; ++o)
#pragma unroll
                for (int i = 0; i < I; ++i)
#pragma unroll
                    for (int j = 0; j < T; ++j) cfma_conj(acc[o][i][j], bj[j], Y[o][i]);
        }
    }
#pragma unroll
    for (int o = 0; o < T; ++o)
#pragma unroll
        for (int i = 0; i < I; ++i)
#pragma unroll
            for (int j = 0; j < T; ++j) {
                const float sx = warp_sum(acc[o][i][j].x), sy = warp_sum(acc[o][i][j].y);
                if (lane == 0 && to0 + o < to_n && t1_0 + i < tr.tau1 && t2_0 + j < tr.tau2) {
                    const int ch = (t1_0 + i) * tr.tau2 + t2_0 + j;
                    const float s = inv[tr.kglob + ch];
                    gW[P.cumW[l] + (int64_t)(to0 + o) * tff + tr.toff + ch] = make_float2(sx * s, sy * s);
                }
            }
}

// weight gradient, depthwise product: warp-task = (triple, t tile, tau_out tile); FF tile generated directly.
template <int T>
__global__ void __launch_bounds__(kGwWarps * kWarp)
fused_gw_dw_kernel(PlanDev P, const int* __restrict__ task_begin, int n_tasks, const float2* __restrict__ Ft,
                   const float2* __restrict__ gOt, const float* __restrict__ inv, float2* __restrict__ gW, int Bp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int task = blockIdx.x * kGwWarps + warp;
    if (task >= n_tasks) return;
    int lo = 0, hi = P.n_triples;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (task_begin[mid] <= task) lo = mid; else hi = mid;
    }
    const TripleRec tr = P.triples[lo];
    const int l = tr.l, n = 2 * l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int to_n = P.tO[l], tff = P.tFF[l];
    const int no = (to_n + T - 1) / T;
    const int r = task - task_begin[lo];
    const int io = r % no, ii = r / no;
    const int t0 = ii * T, to0 = io * T;
    const int G = Bp >> 5;
    float2 acc[T][T];
#pragma unroll
    for (int o = 0; o < T; ++o)
#pragma unroll
        for (int i = 0; i < T; ++i) acc[o][i] = make_float2(0.f, 0.f);
    for (int g = 0; g < G; ++g) {
        const float2* f1 = Ft + ((int64_t)tr.f1off + t0 * n1) * Bp + g * 32 + lane;
        const float2* f2 = Ft + ((int64_t)tr.f2off + t0 * n2) * Bp + g * 32 + lane;
        const float2* go = gOt + (P.cumO[l] + (int64_t)to0 * n) * Bp + g * 32 + lane;
        for (int mi = 0; mi < n; ++mi) {
            float2 v[T];
            gen_tile<T, true>(v, P.cg + tr.cgoff + mi * n2, f1, n1, f2, n2, mi - l, tr.l1, tr.l2, Bp);
#pragma unroll
            for (int o = 0; o < T; ++o) {
                const float2 gv = go[(int64_t)(o * n + mi) * Bp];
#pragma unroll
                for (int i = 0; i < T; ++i) cfma_conj(acc[o][i], v[i], gv);
            }
        }
    }
#pragma unroll
    for (int o = 0; o < T; ++o)
#pragma unroll
        for (int i = 0; i < T; ++i) {
            const float sx = warp_sum(acc[o][i].x), sy = warp_sum(acc[o][i].y);
            if (lane == 0 && to0 + o < to_n && t0 + i < tr.tau1) {
                const float s = inv[tr.kglob + t0 + i];
                gW[P.cumW[l] + (int64_t)(to0 + o) * tff + tr.toff + t0 + i] = make_float2(sx * s, sy * s);
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------
// input gradient.  Block = (fragment lt, kGfOut of its channels, sample group) and owns those elements of gF.  Its
// warps take the fragment's entries (triple, role, tile of the other operand) round-robin; for every m a warp builds
// the gFF tile  g = (1/std) sum_to conj(W[to, k]) gO[to, m]  in registers and contracts it with conj(other operand)
// and C into its private shared-memory accumulator acc[channel][m_t][lane] (CGNet/cudaCG/cudaCG_FNWMM.cu:169-211
// followed by cudaCG_sparse.cu:231-289, without the trip of gFF through memory).
// ---------------------------------------------------------------------------------------------------------------
template <int T, bool DW>
__global__ void __launch_bounds__(kGfWarpsMax * kWarp)
fused_gf_kernel(PlanDev P, const GfEntry* __restrict__ entries, const int* __restrict__ entry_begin,
                const int* __restrict__ block_frag, const float2* __restrict__ Ft, const float2* __restrict__ gOt,
                const float2* __restrict__ W, const float* __restrict__ inv, float2* __restrict__ gF, int B, int Bp) {
    constexpr int OUT = kGfOut;
    constexpr int TI = DW ? 1 : T;   // tile of the other operand
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lt = block_frag[2 * blockIdx.x], t_0 = block_frag[2 * blockIdx.x + 1];
    const int nt = 2 * lt + 1;
    const int g = blockIdx.y;
    const int nwarps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float2* acc = reinterpret_cast<float2*>(smem_raw) + (size_t)warp * OUT * nt * 32;   // [OUT][nt][32]
    for (int i = lane; i < OUT * nt * 32; i += 32) acc[i] = make_float2(0.f, 0.f);
    __syncwarp();
    const int tau_t = P.tF[lt];

    for (int e = entry_begin[lt] + warp; e < entry_begin[lt + 1]; e += nwarps) {
        const GfEntry en = entries[e];
        const TripleRec tr = P.triples[en.triple];
        const int l = tr.l, n = 2 * l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
        const int to_n = P.tO[l], tff = P.tFF[l];
        const float* C = P.cg + tr.cgoff;
        const float2* go = gOt + P.cumO[l] * Bp + g * 32 + lane;
        const float2* Wl = W + P.cumW[l] + tr.toff;
        const bool first = en.role == 0;   // the owned fragment is the first operand of this triple
        // other operand rows
        const int in0 = DW ? t_0 : en.in0;
        const float2* fo = first ? Ft + ((int64_t)tr.f2off + in0 * n2) * Bp + g * 32 + lane
                                 : Ft + ((int64_t)tr.f1off + in0 * n1) * Bp + g * 32 + lane;
        const int tau_o = first ? tr.tau2 : tr.tau1;
        // mid channel and norm factor of every tile entry (out channel a, other channel c)
        int ch[OUT][TI];
        float sc[OUT][TI];
#pragma unroll
        for (int a = 0; a < OUT; ++a)
#pragma unroll
            for (int c = 0; c < TI; ++c) {
                const bool ok = (t_0 + a < tau_t) && (DW || in0 + c < tau_o);
                const int t1 = first ? t_0 + a : in0 + c, t2 = first ? in0 + c : t_0 + a;
                ch[a][c] = ok ? (DW ? t_0 + a : t1 * tr.tau2 + t2) : -1;
                sc[a][c] = ok ? inv[tr.kglob + ch[a][c]] : 0.f;
            }
        for (int mi = 0; mi < n; ++mi) {
            const int m = mi - l;
            float2 gt[OUT][TI];
#pragma unroll
            for (int a = 0; a < OUT; ++a)
#pragma unroll
                for (int c = 0; c < TI; ++c) gt[a][c] = make_float2(0.f, 0.f);
            for (int to = 0; to < to_n; ++to) {
                const float2 gv = go[(int64_t)(to * n + mi) * Bp];
                const float2* w = Wl + (int64_t)to * tff;
#pragma unroll
                for (int a = 0; a < OUT; ++a)
#pragma unroll
                    for (int c = 0; c < TI; ++c)
                        if (ch[a][c] >= 0) cfma_conj(gt[a][c], __ldg(w + ch[a][c]), gv);
            }
#pragma unroll
            for (int a = 0; a < OUT; ++a)
#pragma unroll
                for (int c = 0; c < TI; ++c) {
                    gt[a][c].x *= sc[a][c];
                    gt[a][c].y *= sc[a][c];
                }
            const int lo = max(-tr.l2, m - tr.l1), hi = min(tr.l2, m + tr.l1);
            for (int m2 = lo; m2 <= hi; ++m2) {
                const float cg = C[mi * n2 + m2 + tr.l2];
                // position of the other operand's element and of the owned element along their m axes
                const int mo = first ? (m2 + tr.l2) : (m - m2 + tr.l1);
                const int mt = first ? (m - m2 + tr.l1) : (m2 + tr.l2);
                const int so = first ? n2 : n1;
                float2 x[OUT];
#pragma unroll
                for (int a = 0; a < OUT; ++a) x[a] = make_float2(0.f, 0.f);
                if constexpr (DW) {
                    // depthwise: the other operand's channel is the owned channel itself
#pragma unroll
                    for (int a = 0; a < OUT; ++a)
                        if (ch[a][0] >= 0) {
                            const float2 f = fo[(int64_t)(a * so + mo) * Bp];
                            cfma_conj(x[a], make_float2(f.x * cg, f.y * cg), gt[a][0]);
                        }
                } else {
#pragma unroll
                    for (int c = 0; c < TI; ++c) {
                        float2 f = fo[(int64_t)(c * so + mo) * Bp];
                        f.x *= cg;
                        f.y *= cg;
#pragma unroll
                        for (int a = 0; a < OUT; ++a)
                            if (ch[a][c] >= 0) cfma_conj(x[a], f, gt[a][c]);   // masked entries may hold anything
                    }
                }
#pragma unroll
                for (int a = 0; a < OUT; ++a) {
                    float2* p = acc + (a * nt + mt) * 32 + lane;
                    float2 cur = *p;
                    cur.x += x[a].x;
                    cur.y += x[a].y;
                    *p = cur;
                }
            }
        }
    }
    __syncthreads();
    const float2* all = reinterpret_cast<const float2*>(smem_raw);
    for (int i = threadIdx.x; i < OUT * nt * 32; i += blockDim.x) {
        const int ln = i & 31, rest = i >> 5;
        const int a = rest / nt, mt = rest - a * nt;
        float2 s = make_float2(0.f, 0.f);
        for (int w = 0; w < nwarps; ++w) {
            const float2 v = all[(size_t)w * OUT * nt * 32 + i];
            s.x += v.x;
            s.y += v.y;
        }
        const int b = g * 32 + ln;
        if (b < B && t_0 + a < tau_t) gF[(int64_t)b * P.n_F + P.cumF[lt] + (int64_t)(t_0 + a) * nt + mt] = s;
    }
}

}  // namespace cgb200

using namespace cgb200;

namespace {

struct Workspace {
    float2* Ft;
    float2* Gt;     // gOt in the backward
    float* inv;
    int64_t bytes;
};

int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

// Ft and gOt get kMaxTile*(2*lmax+1) spare rows: masked tile entries read (and discard) rows past a fragment's end.
Workspace carve(const cgb200_plan* p, int64_t B, void* base) {
    const int64_t Bp = (B + 31) / 32 * 32;
    const int64_t pad = (int64_t)kMaxTile * p->max_n;
    Workspace w;
    int64_t off = 0;
    char* c = (char*)base;
    w.Ft = (float2*)(c + off);
    off += align256((p->d.n_F + pad) * Bp * (int64_t)sizeof(float2));
    w.Gt = (float2*)(c + off);
    off += align256((p->d.n_O + pad) * Bp * (int64_t)sizeof(float2));
    w.inv = (float*)(c + off);
    off += align256(std::max<int64_t>(p->d.sum_tff, 1) * (int64_t)sizeof(float));
    w.bytes = off;
    return w;
}

int check_layer(const cgb200_plan* p, int64_t B, const void* ws, int64_t ws_bytes) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    CGB_REQUIRE(p->d.has_out, "the plan was created without tau_out");
    CGB_REQUIRE(B >= 0 && B <= (1ll << 20), "batch size out of range (at most 2^20 samples per call)");
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    CGB_REQUIRE(dev == p->device, "the plan belongs to another CUDA device than the current one");
    if (B > 0) {
        const int64_t need = carve(p, B, nullptr).bytes;
        if (ws == nullptr || ws_bytes < need) {
            set_error("workspace too small: need " + std::to_string(need) + " bytes");
            return CGB200_ERR_WORKSPACE;
        }
        CGB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255) == 0, "workspace must be 256-byte aligned");
    }
    return CGB200_OK;
}

bool al8(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; }

int launch_prep(const PrepJob& a, const PrepJob& b, int njobs, int B, int Bp, const float* stds, float eps, float* inv,
                int n_inv, cudaStream_t st) {
    const int64_t maxN = std::max(a.N, njobs > 1 ? b.N : 0);
    const int gx = (int)std::min<int64_t>((maxN + 31) / 32, 4096);
    launch_begin(K_PREP, st);
    prep_kernel<<<dim3(std::max(gx, 1), Bp / 32, njobs), 256, 0, st>>>(a, b, B, Bp, stds, eps, inv, n_inv);
    launch_end(K_PREP, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // namespace


template <int T>
struct GwI {
    static constexpr int value = T == 1 ? 4 : T == 2 ? 4 : T == 3 ? 3 : T == 4 ? 2 : T == 5 ? 2 : 1;
};

extern "C" {

int64_t cgb200_layer_workspace_bytes(const cgb200_plan* p, int64_t B) {
    if (p == nullptr || B < 0) {
        set_error("null plan or negative batch");
        return -1;
    }
    return carve(p, std::max<int64_t>(B, 1), nullptr).bytes;
}

int cgb200_layer_fwd(const cgb200_plan* p, const float* F, const float* W, float* stds, float cnt, float eps, int flags,
                     float* O, int64_t B, void* workspace, int64_t workspace_bytes, void* stream) {
    int rc = check_layer(p, B, workspace, workspace_bytes);
    if (rc) return rc;
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    const bool update = fn && (flags & CGB200_FN_UPDATE);
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    if (B == 0 || p->d.n_O == 0) return CGB200_OK;
    CGB_REQUIRE(F != nullptr && O != nullptr && (W != nullptr || p->d.w_len == 0), "null buffer");
    CGB_REQUIRE(al8(F) && al8(W) && al8(O), "buffers must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int Bp = (int)((B + 31) / 32 * 32);
    Workspace ws = carve(p, B, workspace);

    PrepJob jf{(const float2*)F, ws.Ft, p->d.n_F}, none{nullptr, nullptr, 0};
    if ((rc = launch_prep(jf, none, 1, (int)B, Bp, fn ? stds : nullptr, eps, update ? nullptr : ws.inv, p->d.sum_tff, st)))
        return rc;
    if (update && p->d.n_cells > 0) {
        launch_begin(K_STATS, st);
        CGB_DISPATCH_TILE(p->d.tile, p->d.depthwise,
                          (fused_stats_kernel<TT, DD><<<p->d.n_cells, 256, 0, st>>>(p->d, ws.Ft, stds, ws.inv, cnt, eps, (int)B, Bp)));
        launch_end(K_STATS, st);
        CGB_CUDA(cudaGetLastError());
    }
    const dim3 grid((p->d.lmax + 1) * (p->d.lmax + 1), Bp / 32);
    launch_begin(K_FWD, st);
    CGB_DISPATCH_TILE(p->d.tile, p->d.depthwise,
                      (fused_fwd_kernel<TT, DD><<<grid, kFwdWarps * kWarp, 0, st>>>(p->d, ws.Ft, (const float2*)W, ws.inv, (float2*)O, (int)B, Bp)));
    launch_end(K_FWD, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

int cgb200_layer_bwd(const cgb200_plan* p, const float* F, const float* W, const float* stds, float eps, int flags,
                     const float* gO, float* gF, float* gW, int64_t B, void* workspace, int64_t workspace_bytes,
                     void* stream) {
    int rc = check_layer(p, B, workspace, workspace_bytes);
    if (rc) return rc;
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    CGB_REQUIRE(al8(F) && al8(W) && al8(gO) && al8(gF) && al8(gW), "buffers must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        if (p->d.w_len > 0) {
            CGB_REQUIRE(gW != nullptr, "gW is null");
            CGB_CUDA(cudaMemsetAsync(gW, 0, p->d.w_len * sizeof(float2), st));
        }
        return CGB200_OK;
    }
    CGB_REQUIRE(F != nullptr && gF != nullptr && (gO != nullptr || p->d.n_O == 0), "null buffer");
    CGB_REQUIRE(p->d.w_len == 0 || (W != nullptr && gW != nullptr), "W or gW is null");
    const int Bp = (int)((B + 31) / 32 * 32);
    Workspace ws = carve(p, B, workspace);

    PrepJob jf{(const float2*)F, ws.Ft, p->d.n_F}, jg{(const float2*)gO, ws.Gt, p->d.n_O};
    if ((rc = launch_prep(jf, jg, p->d.n_O > 0 ? 2 : 1, (int)B, Bp, fn ? stds : nullptr, eps, ws.inv, p->d.sum_tff, st))) return rc;

    // weight gradient
    const int n_tasks = p->gw_begin.empty() ? 0 : p->gw_begin.back();
    if (n_tasks > 0) {
        const int blocks = (n_tasks + kGwWarps - 1) / kGwWarps;
        launch_begin(K_GW, st);
        if (p->d.depthwise) {
            CGB_DISPATCH_TILE(p->d.tile, false,
                              (fused_gw_dw_kernel<TT><<<blocks, kGwWarps * kWarp, 0, st>>>(p->d, p->d_gw_begin, n_tasks, ws.Ft, ws.Gt, ws.inv, (float2*)gW, Bp)));
        } else {
            CGB_DISPATCH_TILE(p->d.tile, false,
                              (fused_gw_kernel<TT, GwI<TT>::value><<<blocks, kGwWarps * kWarp, 0, st>>>(p->d, p->d_gw_begin, n_tasks, ws.Ft, ws.Gt, ws.inv, (float2*)gW, Bp)));
        }
        launch_end(K_GW, st);
        CGB_CUDA(cudaGetLastError());
    }
    // degrees with output channels but no mid channels have no weights; every other weight was written above

    // input gradient
    if (p->d.n_F > 0) {
        const int nblk = (int)p->gf_blocks.size() / 2;
        const size_t per_warp = (size_t)kGfOut * p->max_n * 32 * sizeof(float2);
        int nwarps = (int)std::min<size_t>(kGfWarpsMax, (200 * 1024) / per_warp);
        if (nwarps < 1) {
            set_error("lmax too large for the fused input-gradient kernel");
            return CGB200_ERR_UNSUPPORTED;
        }
        const size_t smem = per_warp * nwarps;
        launch_begin(K_GF, st);
        CGB_DISPATCH_TILE(p->d.tile, p->d.depthwise, {
            auto kern = fused_gf_kernel<TT, DD>;
            if (smem > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<dim3(nblk, Bp / 32), nwarps * kWarp, smem, st>>>(p->d, p->d_gf_entries, p->d_gf_begin, p->d_gf_blocks, ws.Ft, ws.Gt, (const float2*)W, ws.inv, (float2*)gF, (int)B, Bp);
        });
        launch_end(K_GF, st);
        CGB_CUDA(cudaGetLastError());
    }
    return CGB200_OK;
}

}  // extern "C"
