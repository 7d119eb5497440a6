// The whole CG layer without a materialised mid activation: cgb200_layer_fwd / cgb200_layer_bwd.
//
// Layout idea: the activations are first rearranged into "slabs" (see PlanDev): samples in groups of 32, one sample
// per lane, and inside a group every fragment stored tile-interleaved, [channel tile][m][channel in tile][32 lanes].
// A warp works on one group, so everything except the sample is uniform across it: the (l, l1, l2, m, m2) band loops
// never diverge, CG coefficients, mixing weights and norm factors are warp-uniform loads, operand loads are whole
// 256-byte lines whose offsets inside the inner loops are compile-time constants, and the sums over the batch that the
// statistics and the weight gradient need are fixed-order warp-shuffle trees.  No float atomics anywhere: every output
// element has exactly one owner and every sum a fixed order, so results are bit-identical from run to run.
//
//   prep          F (and gO) -> slabs; 1/max(eps, std) per mid channel when the statistics are not being updated
//   stats         training only: per mid channel std of |FF| over (b, m) from on-the-fly FF; moving average; 1/max(eps,.)
//   fwd           O[b, l, :, m] = sum over the cells of degree l of  W_l[:, k] * (FF[b, k, m] / std_k)
//                 two variants: rows (l, m) as independent blocks reading the slab through L1, or - when a group's
//                 whole slab fits in shared memory - persistent blocks that stage the slab once and pull rows from a
//                 cost-sorted queue
//   grad_w        gW_l[to, (t1,t2)] = (1/std) sum_{b, m2} conj(F2[t2, m2]) * sum_m C[m, m2] conj(F1[t1, m-m2]) gO[to, m]
//   grad_f        gF via gFF tiles built from gO and W in registers, contracted with conj(F) and C into per-warp
//                 shared-memory accumulators that one block owns
#include <cuda_pipeline.h>
#include <algorithm>

#include "common.cuh"

namespace cgb200 {

constexpr int kWarp = 32;
constexpr int kFwdWarps = 8;      // warps of a forward block = slices of the degree's cell list
constexpr int kFwdTo = 16;        // output channels accumulated in registers per pass
constexpr int kSlabWarps = 16;    // warps of a persistent forward block
constexpr int kGwWarps = 4;

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
// prep: up to two rearrangements src[B][N] -> slab in one launch (blockIdx.z picks the job), the norm factors, and the
// reset of the forward kernel's row counters.
// ---------------------------------------------------------------------------------------------------------------
struct PrepJob {
    const float2* src;     // [B][N]
    float2* dst;           // [G][nS][32]
    int64_t N;
    const int64_t* cum;    // [lmax+2] fragment starts in src
    const int* cumS;       // [lmax+2] fragment starts in the slab
    const int* tau;        // [lmax+1]
    int nS;
    int has_pad;           // some fragment's channel count is not a multiple of the tile
};

__global__ void __launch_bounds__(256)
prep_kernel(PrepJob j0, PrepJob j1, int lmax, int T, int B, const float* __restrict__ stds, float eps,
            float* __restrict__ inv, int n_inv, int* __restrict__ counters, int n_counters) {
    __shared__ float2 tile[32][33];
    const PrepJob job = blockIdx.z == 0 ? j0 : j1;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t flat_block = (int64_t)blockIdx.y * gridDim.x + blockIdx.x;
    if (blockIdx.z == 0) {
        const int64_t stride = (int64_t)gridDim.x * gridDim.y * 256;
        if (inv != nullptr)
            for (int64_t k = flat_block * 256 + threadIdx.x; k < n_inv; k += stride)
                inv[k] = stds ? 1.f / fmaxf(eps, stds[k]) : 1.f;
        if (flat_block == 0)
            for (int k = threadIdx.x; k < n_counters; k += 256) counters[k] = 0;
    }
    const int g = blockIdx.y;
    float2* dst = job.dst + (int64_t)g * job.nS * 32;
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
            if (e < job.N) {
                const int l = find_degree(job.cum, lmax + 1, e);
                const int n = 2 * l + 1;
                const int r = (int)(e - job.cum[l]);
                const int t = r / n, mi = r - t * n;
                const int es = job.cumS[l] + ((t / T) * n + mi) * T + t % T;
                dst[(int64_t)es * 32 + tx] = tile[tx][ty + 8 * k];
            }
        }
    }
    if (job.has_pad) {   // zero the channels that pad a fragment to whole tiles
        for (int es = blockIdx.x * 8 + ty; es < job.nS; es += gridDim.x * 8) {
            int lo = 0, hi = lmax + 1;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (job.cumS[mid] <= es) lo = mid; else hi = mid;
            }
            const int n = 2 * lo + 1;
            const int r = es - job.cumS[lo];
            const int t = (r / (T * n)) * T + r % T;
            if (t >= job.tau[lo]) dst[(int64_t)es * 32 + tx] = make_float2(0.f, 0.f);
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

// Body of the statistics kernel for the tile entries [E0, E0 + NE): the whole tile, or (full product, SPLIT) the rows
// I0 .. I0+IN of it, in which case two blocks share a cell and each needs half the registers, so that two blocks fit an SM.
template <int T, bool DW, int I0, int IN>
__device__ __forceinline__ void stats_body(const PlanDev& P, const CellRec& cell, const TripleRec& tr, const float2* __restrict__ SF,
                                           float* __restrict__ stds, float* __restrict__ inv, float cnt, float eps, int B, int G,
                                           const float* __restrict__ C, double (*red)[TileShape<T, DW>::NV][2],
                                           float2* __restrict__ ff_tile = nullptr, int64_t ff_stride = 0) {
    constexpr int NE = DW ? IN : IN * T;      // tile entries handled here
    constexpr int E0 = DW ? I0 : I0 * T;      // first of them
    const int n = 2 * tr.l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float s1[NE], s1c[NE], s2[NE];
#pragma unroll
    for (int i = 0; i < NE; ++i) s1[i] = s1c[i] = s2[i] = 0.f;
    const int o1 = P.cumSF[tr.l1] + (cell.t1_0 / T) * n1 * T, o2 = P.cumSF[tr.l2] + (cell.t2_0 / T) * n2 * T;
    for (int task = warp; task < G * n; task += 8) {
        const int g = task / n, mi = task - g * n;
        const float2* slab = SF + (int64_t)g * P.nSF * 32 + lane;
        float2 v[NE];
        if constexpr (!DW && IN < T) gen_slab_rows<T, I0, IN>(v, C + mi * n2, slab + o1 * 32, slab + o2 * 32, mi - tr.l, tr.l1, tr.l2);
        else gen_slab<T, DW, true>(v, C + mi * n2, slab + o1 * 32, slab + o2 * 32, mi - tr.l, tr.l1, tr.l2);
        if constexpr (!DW) {
            if (ff_tile != nullptr) {   // keep the tile for the forward that follows: [group][cell][m][entry][lane]
                float2* dst = ff_tile + ((int64_t)g * ff_stride + (int64_t)mi * (T * T) + E0) * 32 + lane;
#pragma unroll
                for (int i = 0; i < NE; ++i) dst[i * 32] = v[i];
            }
        }
#pragma unroll
        for (int i = 0; i < NE; ++i) {
            const float nrm = v[i].x * v[i].x + v[i].y * v[i].y;
            const float r = sqrtf(nrm);
            s2[i] += nrm;
            s1[i] += r;
            if (nrm > 0.f) s1c[i] += __fdividef(0.5f * fmaf(-r, r, nrm), r);
        }
    }
#pragma unroll
    for (int i = 0; i < NE; ++i) {
        const double a = warp_sum((double)s1[i] + (double)s1c[i]), b = warp_sum((double)s2[i]);
        if (lane == 0) {
            red[warp][i][0] = a;
            red[warp][i][1] = b;
        }
    }
    __syncthreads();
    const int idx = threadIdx.x;
    if (idx < NE && tile_valid<T, DW>(E0 + idx, cell.t1_0, cell.t2_0, tr.tau1, tr.tau2)) {
        double m1 = 0.0, m2 = 0.0;
        for (int w = 0; w < 8; ++w) {
            m1 += red[w][idx][0];
            m2 += red[w][idx][1];
        }
        const double N = (double)B * n;
        const double var = m2 / N - (m1 / N) * (m1 / N);
        const double sigma = var > 0.0 ? sqrt(var) : 0.0;
        const int k = tr.kglob + tile_channel<T, DW>(E0 + idx, cell.t1_0, cell.t2_0, tr.tau2);
        const float s = moving_std_f(stds[k], sigma, cnt);
        stds[k] = s;
        inv[k] = 1.f / fmaxf(eps, s);
    }
}

// grid = cells, or 2 x cells with SPLIT (block 2c handles the first ceil(T/2) rows of cell c's tile, block 2c+1 the rest)
template <int T, bool DW, bool SPLIT>
__global__ void __launch_bounds__(256, (SPLIT || T <= 4) ? 2 : 1)
fused_stats_kernel(PlanDev P, const float2* __restrict__ SF, float* __restrict__ stds, float* __restrict__ inv, float cnt,
                   float eps, int B, int G, float2* __restrict__ ff, int64_t ff_stride, const int64_t* __restrict__ ff_off) {
    constexpr int NV = TileShape<T, DW>::NV;
    __shared__ double red[8][NV][2];
    extern __shared__ __align__(16) float sband[];   // the triple's CG band, (2l+1) x (2l2+1)
    const int blk = SPLIT ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int cidx = P.n_cells - 1 - blk;            // the last degrees carry the long bands: start them first
    const CellRec cell = P.cells[cidx];
    const TripleRec tr = P.triples[cell.triple];
    const int n = 2 * tr.l + 1, n2 = 2 * tr.l2 + 1;
    for (int i = threadIdx.x; i < n * n2; i += 256) sband[i] = P.cg[tr.cgoff + i];
    __syncthreads();
    // ff: the generated tiles are also written out (full product), so that the forward that follows reads them back
    // instead of generating them again
    float2* tile = (DW || ff == nullptr || P.tO[tr.l] == 0) ? nullptr : ff + (ff_off[tr.l] + (int64_t)(cidx - P.cell_begin[tr.l]) * n * TileShape<T, DW>::NV) * 32;
    if constexpr (SPLIT && !DW && T > 1) {
        constexpr int AH = (T + 1) / 2;
        if ((blockIdx.x & 1) == 0) stats_body<T, DW, 0, AH>(P, cell, tr, SF, stds, inv, cnt, eps, B, G, sband, red, tile, ff_stride);
        else stats_body<T, DW, AH, T - AH>(P, cell, tr, SF, stds, inv, cnt, eps, B, G, sband, red, tile, ff_stride);
    } else {
        stats_body<T, DW, 0, T>(P, cell, tr, SF, stds, inv, cnt, eps, B, G, sband, red, tile, ff_stride);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// forward.  One output row = (degree l, m) for one sample group.  The warps of a block take the cells of the degree
// round-robin, each lane keeps up to kFwdTo output channels of its sample in registers, and the warps' partial sums
// are added in warp order.  `slab` is this lane's view of the group's input slab (global or shared memory).
// ---------------------------------------------------------------------------------------------------------------
// Per-warp staging area of the forward kernels: the mixing-weight tile of a cell, its norm factors and the CG band row
// of its (cell, m), fetched by the lanes together and then read back as broadcasts (without it every one of those
// warp-uniform values is a dependent load at L2 latency).  Two buffers per warp: the next cell's values arrive by
// asynchronous copies while the current cell is computed.
__host__ __device__ inline int fwd_stage_half_bytes(int step, int nv, int max_n) {
    return ((step * nv * 8 + nv * 4 + max_n * 4) + 15) & ~15;
}
__host__ __device__ inline int fwd_stage_bytes(int step, int nv, int max_n) { return 2 * fwd_stage_half_bytes(step, nv, max_n); }

// (`tiles`: this lane's view of the group's kept tiles, written by the statistics kernel of the same call, or null;
// their values are what gen_slab would produce, bit for bit.)
template <int T, bool DW, int NW, int NTO>
__device__ __forceinline__ void fwd_row(const PlanDev& P, const float2* __restrict__ slab, const float2* __restrict__ W,
                                        const float* __restrict__ inv, float2* __restrict__ O, float2* __restrict__ red,
                                        unsigned char* __restrict__ stage, int l, int mi, int b, int B, int warp, int lane,
                                        const float2* __restrict__ tiles, const int64_t* __restrict__ ff_off) {
    constexpr int NV = TileShape<T, DW>::NV;
    const int n = 2 * l + 1;
    const int to_n = P.tO[l];
    const int tff = P.tFF[l];
    const int c_begin = P.cell_begin[l], c_end = P.cell_begin[l + 1];
    const float2* Wl = W + P.cumW[l];
    constexpr int step = NTO;   // output channels per pass, a compile-time constant so that no issue slot is wasted
    constexpr int red_to = NTO;
    const int half = fwd_stage_half_bytes(step, NV, P.lmax * 2 + 1);
    for (int to0 = 0; to0 < to_n; to0 += step) {
        float2 o[NTO];
#pragma unroll
        for (int t = 0; t < NTO; ++t) o[t] = make_float2(0.f, 0.f);
        // asynchronous copies of one cell's tile of W (zero where the tile or the pass has no channel), its norm factors
        // and its band row into one of the warp's two staging buffers
        auto stage_cell = [&](const CellInfo& x, unsigned char* st) {
            float2* wb = reinterpret_cast<float2*>(st);          // [step][NV]
            float* ib = reinterpret_cast<float*>(wb + step * NV);  // [NV]
            float* cb = ib + NV;                                   // [2*l2+1]
            const int xn2 = 2 * x.l2 + 1;
            for (int e = lane; e < step * NV; e += 32) {
                const int t = e / NV, idx = e - t * NV;
                const int i = DW ? idx : idx / T, j = DW ? 0 : idx % T;
                const bool ok = (i < x.v1) && (DW || j < x.v2) && (to0 + t < to_n);
                const float2* src = ok ? Wl + (int64_t)(to0 + t) * tff + x.wch0 + (DW ? i : i * x.tau2 + j) : Wl;
                __pipeline_memcpy_async(wb + e, src, 8, ok ? 0 : 8);
            }
            for (int idx = lane; idx < NV; idx += 32) {
                const int i = DW ? idx : idx / T, j = DW ? 0 : idx % T;
                const bool ok = (i < x.v1) && (DW || j < x.v2);
                __pipeline_memcpy_async(ib + idx, ok ? inv + x.kch0 + (DW ? i : i * x.tau2 + j) : inv, 4, ok ? 0 : 4);
            }
            for (int e = lane; e < xn2; e += 32) __pipeline_memcpy_async(cb + e, P.cg + x.cgoff + mi * xn2 + e, 4);
            __pipeline_commit();
        };
        int c = c_begin + warp;
        int buf = 0;
        CellInfo ci, nx;
        __syncwarp();   // the previous pass's readers are done with the staging area
        if (c < c_end) {
            ci = P.cell_info[c];
            stage_cell(ci, stage);
            if (c + NW < c_end) nx = P.cell_info[c + NW];
        }
        while (c < c_end) {
            const int cn = c + NW;
            const bool has_next = cn < c_end;
            CellInfo nx2;
            if (cn + NW < c_end) nx2 = P.cell_info[cn + NW];   // two cells ahead: in flight while this cell is computed
            if (has_next) stage_cell(nx, stage + (buf ^ 1) * half);
            if (has_next) __pipeline_wait_prior(1); else __pipeline_wait_prior(0);   // this cell's copies have landed
            __syncwarp();
            const float2* wbuf = reinterpret_cast<const float2*>(stage + buf * half);
            const float* ibuf = reinterpret_cast<const float*>(wbuf + step * NV);
            const float* cbuf = ibuf + NV;
            float2 v[NV];
            if (!DW && tiles != nullptr) {
                const float2* src = tiles + (ff_off[l] + ((int64_t)(c - c_begin) * n + mi) * NV) * 32;
#pragma unroll
                for (int idx = 0; idx < NV; ++idx) v[idx] = src[idx * 32];
            } else {
                gen_slab<T, DW>(v, cbuf, slab + ci.o1 * 32, slab + ci.o2 * 32, mi - l, ci.l1, ci.l2);
            }
#pragma unroll
            for (int idx = 0; idx < NV; ++idx) {
                const float sc = ibuf[idx];
                const float2 x = make_float2(v[idx].x * sc, v[idx].y * sc);
#pragma unroll
                for (int t = 0; t < NTO; ++t) cfma(o[t], wbuf[t * NV + idx], x);   // masked entries carry zero weights
            }
            __syncwarp();   // every lane is done with this buffer before the next iteration's copies overwrite it
            ci = nx;
            nx = nx2;
            c = cn;
            buf ^= 1;
        }
        __syncthreads();   // protects `red` from the previous pass / row
#pragma unroll
        for (int t = 0; t < NTO; ++t) red[(warp * red_to + t) * 32 + lane] = o[t];
        __syncthreads();
        for (int t = warp; t < step && to0 + t < to_n; t += NW) {
            float2 s = red[t * 32 + lane];
            for (int w = 1; w < NW; ++w) {
                const float2 q = red[(w * red_to + t) * 32 + lane];
                s.x += q.x;
                s.y += q.y;
            }
            if (b < B) O[(int64_t)b * P.n_O + P.cumO[l] + (int64_t)(to0 + t) * n + mi] = s;
        }
    }
}

// rows as independent blocks; the slab is read through L1.  grid = (rows, groups)
template <int T, bool DW, int NTO>
__global__ void __launch_bounds__(kFwdWarps * kWarp)
fused_fwd_kernel(PlanDev P, const int* __restrict__ rows, const float2* __restrict__ SF, const float2* __restrict__ W,
                 const float* __restrict__ inv, float2* __restrict__ O, int B, int stage_bytes, const float2* __restrict__ ff,
                 int64_t ff_stride, const int64_t* __restrict__ ff_off) {
    constexpr int red_to = NTO;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* red = reinterpret_cast<float2*>(smem_raw);
    const int l = rows[2 * blockIdx.x], mi = rows[2 * blockIdx.x + 1];
    const int g = blockIdx.y;   // group-major block order: consecutive blocks on an SM read the same group's slab through L1
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* stage = smem_raw + (size_t)kFwdWarps * red_to * 32 * sizeof(float2) + (size_t)warp * stage_bytes;
    fwd_row<T, DW, kFwdWarps, NTO>(P, SF + (int64_t)g * P.nSF * 32 + lane, W, inv, O, red, stage, l, mi, g * 32 + lane, B, warp,
                                   lane, ff == nullptr ? nullptr : ff + (int64_t)g * ff_stride * 32 + lane, ff_off);
}

// persistent blocks: block (p, g) copies group g's slab into shared memory once, then pulls rows (most expensive
// first) from the group's counter until none is left.  grid = (blocks per group, groups)
template <int T, bool DW, int NTO>
__global__ void __launch_bounds__(kSlabWarps * kWarp)
fused_fwd_slab_kernel(PlanDev P, const int* __restrict__ rows, int n_rows, const float2* __restrict__ SF,
                      const float2* __restrict__ W, const float* __restrict__ inv, float2* __restrict__ O, int B,
                      int* __restrict__ counters, int stage_bytes, const float2* __restrict__ ff, int64_t ff_stride,
                      const int64_t* __restrict__ ff_off) {
    constexpr int red_to = NTO;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int next_row;
    float2* slab = reinterpret_cast<float2*>(smem_raw);
    float2* red = slab + (size_t)P.nSF * 32;
    unsigned char* stage = reinterpret_cast<unsigned char*>(red + (size_t)kSlabWarps * red_to * 32) +
                           (size_t)(threadIdx.x >> 5) * stage_bytes;
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const float4* src = reinterpret_cast<const float4*>(SF + (int64_t)g * P.nSF * 32);
        float4* dst = reinterpret_cast<float4*>(slab);
        for (int i = threadIdx.x; i < P.nSF * 16; i += blockDim.x) dst[i] = src[i];
    }
    for (;;) {
        __syncthreads();   // slab staged / previous row finished with next_row
        if (threadIdx.x == 0) next_row = atomicAdd(counters + g, 1);
        __syncthreads();
        const int r = next_row;
        if (r >= n_rows) break;
        fwd_row<T, DW, kSlabWarps, NTO>(P, slab + lane, W, inv, O, red, stage, rows[2 * r], rows[2 * r + 1], g * 32 + lane, B, warp,
                                        lane, ff == nullptr ? nullptr : ff + (int64_t)g * ff_stride * 32 + lane, ff_off);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// weight gradient, full product.  Warp-task = (triple, I consecutive t1 inside one tile, one t2 tile, one tau_out
// tile).  A lane keeps acc[o][i][j] for its own sample; the sample groups are visited in order and the lanes summed at
// the end.  The task list is sorted by cost, most expensive first, so the blocks that start first carry the long bands
// and the cheap tasks fill the tail.
// ---------------------------------------------------------------------------------------------------------------
// One task of the weight-gradient kernel with exactly I rows of t1.
// `last_rep` > 1: the last sample group holds at most 32 / last_rep samples.  Its lanes are then (sample, j) pairs,
// sample = lane % (32 / last_rep), and lane group j takes the values m2 = -l2 + j, -l2 + j + last_rep, ... of the outer
// loop instead of every lane walking all of them for an empty sample slot: the group costs 1 / last_rep of a full one
// (plus what the lanes' different band lengths cost in divergence).  The warp-wide sum at the end adds the lane groups up.
template <int T, int I, int TO>
__device__ __forceinline__ void gw_unit(const PlanDev& P, const GwTask tk, int slice, int slices, const float2* __restrict__ SF,
                                        const float2* __restrict__ SG, const float* __restrict__ inv, float2* __restrict__ out,
                                        int G, float* __restrict__ band, int lane, int last_rep) {
    const TripleRec tr = P.triples[tk.triple];
    const int l = tr.l, n = 2 * l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int to_n = P.tO[l], tff = P.tFF[l];
    const int q1 = tk.q1, q2 = tk.q2, qo = tk.qo;
    const int j0 = tk.gi;   // first t1 row of the task inside its tile; the task covers exactly I rows
    __syncwarp();   // the previous task's readers are done with the band
    for (int e = lane; e < n * n2; e += 32) band[e] = __ldg(P.cg + tr.cgoff + e);
    __syncwarp();
    const float* C = band;
    int jrow[I];   // channel inside the tile read for row i (clamped: rows past the tile are masked at the end)
#pragma unroll
    for (int i = 0; i < I; ++i) jrow[i] = min(j0 + i, T - 1);
    int goff[TO];  // slab offset of output channel qo*TO+o at m index 0 (clamped to the last channel, masked at the end)
#pragma unroll
    for (int o = 0; o < TO; ++o) {
        const int to = min(qo * TO + o, to_n - 1);
        goff[o] = ((to / T) * n * T + to % T) * 32;
    }

    float2 acc[TO][I][T];
#pragma unroll
    for (int o = 0; o < TO; ++o)
#pragma unroll
        for (int i = 0; i < I; ++i)
#pragma unroll
            for (int j = 0; j < T; ++j) acc[o][i][j] = make_float2(0.f, 0.f);

    for (int g = slice; g < G; g += slices) {
        const int rep = (g == G - 1) ? last_rep : 1;         // warp-uniform
        const int slot = rep > 1 ? lane % (32 / rep) : lane;   // this lane's sample inside the group
        const int m2_first = -tr.l2 + (rep > 1 ? lane / (32 / rep) : 0);
        const float2* f1 = SF + ((int64_t)g * P.nSF + P.cumSF[tr.l1] + q1 * n1 * T) * 32 + slot;
        const float2* f2 = SF + ((int64_t)g * P.nSF + P.cumSF[tr.l2] + q2 * n2 * T) * 32 + slot;
        const float2* go = SG + ((int64_t)g * P.nSO + P.cumSO[l]) * 32 + slot;
        for (int m2 = m2_first; m2 <= tr.l2; m2 += rep) {
            float2 Y[TO][I];
#pragma unroll
            for (int o = 0; o < TO; ++o)
#pragma unroll
                for (int i = 0; i < I; ++i) Y[o][i] = make_float2(0.f, 0.f);
            const int mlo = max(-l, m2 - tr.l1), mhi = min(l, m2 + tr.l1);
            const float* pc = C + (mlo + l) * n2 + m2 + tr.l2;
            const float2* p1 = f1 + (mlo - m2 + tr.l1) * (T * 32);
            const float2* pg = go + (mlo + l) * (T * 32);
            // software pipeline: the operands of band step k+1 are in flight while step k's FMAs run (the last step
            // fetches its own again); they come from global memory through L1
            if (mhi >= mlo) {
                float c = *pc;
                float2 a[I], gv[TO];
#pragma unroll
                for (int i = 0; i < I; ++i) a[i] = p1[jrow[i] * 32];
#pragma unroll
                for (int o = 0; o < TO; ++o) gv[o] = pg[goff[o]];
                for (int k = mhi - mlo; k >= 0; --k) {
                    const int adv = k > 0 ? 1 : 0;
                    pc += adv * n2;
                    p1 += adv * (T * 32);
                    pg += adv * (T * 32);
                    const float cn = *pc;
                    float2 an[I], gn[TO];
#pragma unroll
                    for (int i = 0; i < I; ++i) an[i] = p1[jrow[i] * 32];
#pragma unroll
                    for (int o = 0; o < TO; ++o) gn[o] = pg[goff[o]];
#pragma unroll
                    for (int i = 0; i < I; ++i) {
                        a[i].x *= c;
                        a[i].y *= c;
                    }
#pragma unroll
                    for (int o = 0; o < TO; ++o)
#pragma unroll
                        for (int i = 0; i < I; ++i) cfma_conj(Y[o][i], a[i], gv[o]);
                    c = cn;
#pragma unroll
                    for (int i = 0; i < I; ++i) a[i] = an[i];
#pragma unroll
                    for (int o = 0; o < TO; ++o) gv[o] = gn[o];
                }
            }
            const float2* p2 = f2 + (m2 + tr.l2) * (T * 32);
            float2 bj[T];
#pragma unroll
            for (int j = 0; j < T; ++j) bj[j] = p2[j * 32];
#pragma unroll
            for (int o = 0; o < TO; ++o)
#pragma unroll
                for (int i = 0; i < I; ++i)
#pragma unroll
                    for (int j = 0; j < T; ++j) cfma_conj(acc[o][i][j], bj[j], Y[o][i]);
        }
    }
#pragma unroll
    for (int o = 0; o < TO; ++o)
#pragma unroll
        for (int i = 0; i < I; ++i)
#pragma unroll
            for (int j = 0; j < T; ++j) {
                const float sx = warp_sum(acc[o][i][j].x), sy = warp_sum(acc[o][i][j].y);
                const int t1 = q1 * T + j0 + i, t2 = q2 * T + j, to = qo * TO + o;
                if (lane == 0 && j0 + i < T && to < to_n && t1 < tr.tau1 && t2 < tr.tau2) {
                    const int ch = t1 * tr.tau2 + t2;
                    const float s = inv[tr.kglob + ch];
                    out[P.cumW[l] + (int64_t)to * tff + tr.toff + ch] = make_float2(sx * s, sy * s);
                }
            }
}

template <int T, int TO>
__global__ void __launch_bounds__(kGwWarps * kWarp, 3)
fused_gw_kernel(PlanDev P, const GwTask* __restrict__ tasks, int n_tasks, const float2* __restrict__ SF,
                const float2* __restrict__ SG, const float* __restrict__ inv, float2* __restrict__ gW, int G,
                int band_floats, int slices, int64_t slice_stride, int last_rep) {
    extern __shared__ __align__(16) float sband_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* band = sband_all + (size_t)warp * band_floats;   // this warp's copy of the current triple's CG band
    // unit = (task, slice): slice s sums the sample groups s, s + slices, ...; with more than one slice the partial
    // sums go to gW + s * slice_stride and gw_reduce_kernel adds them in slice order
    for (int unit = blockIdx.x * kGwWarps + warp; unit < n_tasks * slices; unit += gridDim.x * kGwWarps) {
        const int task = unit / slices, slice = unit - task * slices;
        float2* __restrict__ out = gW + (int64_t)slice * slice_stride;
        const GwTask tk = tasks[task];
        // the row groups of a tile are exact (GwRows): a task has GwRows<T>::A rows or, for the last group of a tile
        // whose edge is not a multiple of A, GwRows<T>::B rows
        if (tk.ni == GwRows<T>::A) gw_unit<T, GwRows<T>::A, TO>(P, tk, slice, slices, SF, SG, inv, out, G, band, lane, last_rep);
        if constexpr (GwRows<T>::B > 0)
            if (tk.ni == GwRows<T>::B) gw_unit<T, GwRows<T>::B, TO>(P, tk, slice, slices, SF, SG, inv, out, G, band, lane, last_rep);
    }
}

// gW[i] = sum over the slices, in slice order
__global__ void __launch_bounds__(256)
gw_reduce_kernel(const float2* __restrict__ partial, int slices, int64_t slice_stride, float2* __restrict__ gW, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float2 s = partial[i];
        for (int k = 1; k < slices; ++k) {
            const float2 v = partial[(int64_t)k * slice_stride + i];
            s.x += v.x;
            s.y += v.y;
        }
        gW[i] = s;
    }
}

void launch_gw_reduce(const cgb200_plan* p, const float2* partial, int slices, float2* gW, cudaStream_t st) {
    launch_begin(K_GW_REDUCE, st);
    const int gx = (int)std::min<int64_t>((p->d.w_len + 255) / 256, 4 * p->num_sms);
    gw_reduce_kernel<<<gx, 256, 0, st>>>(partial, slices, p->d.w_len, gW, p->d.w_len);
    launch_end(K_GW_REDUCE, st);
}

// weight gradient, depthwise product: warp-task = (triple, t tile, tau_out tile); FF tile generated directly.
template <int T>
__global__ void __launch_bounds__(kGwWarps * kWarp)
fused_gw_dw_kernel(PlanDev P, const GwTask* __restrict__ tasks, int n_tasks, const float2* __restrict__ SF,
                   const float2* __restrict__ SG, const float* __restrict__ inv, float2* __restrict__ gW, int G,
                   int band_floats) {
    extern __shared__ __align__(16) float sband_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int task = blockIdx.x * kGwWarps + warp;   // the task list is sorted, most expensive first
    if (task >= n_tasks) return;
    const GwTask tk = tasks[task];
    const TripleRec tr = P.triples[tk.triple];
    const int l = tr.l, n = 2 * l + 1, n1 = 2 * tr.l1 + 1, n2 = 2 * tr.l2 + 1;
    const int to_n = P.tO[l], tff = P.tFF[l];
    const int qo = tk.qo, q = tk.q1;
    float* band = sband_all + (size_t)warp * band_floats;
    for (int e = lane; e < n * n2; e += 32) band[e] = __ldg(P.cg + tr.cgoff + e);
    __syncwarp();
    float2 acc[T][T];
#pragma unroll
    for (int o = 0; o < T; ++o)
#pragma unroll
        for (int i = 0; i < T; ++i) acc[o][i] = make_float2(0.f, 0.f);
    for (int g = 0; g < G; ++g) {
        const float2* f1 = SF + ((int64_t)g * P.nSF + P.cumSF[tr.l1] + q * n1 * T) * 32 + lane;
        const float2* f2 = SF + ((int64_t)g * P.nSF + P.cumSF[tr.l2] + q * n2 * T) * 32 + lane;
        const float2* go = SG + ((int64_t)g * P.nSO + P.cumSO[l] + qo * n * T) * 32 + lane;
        for (int mi = 0; mi < n; ++mi) {
            float2 v[T];
            gen_slab<T, true>(v, band + mi * n2, f1, f2, mi - l, tr.l1, tr.l2);
#pragma unroll
            for (int o = 0; o < T; ++o) {
                const float2 gv = go[(mi * T + o) * 32];
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
            const int t = q * T + i, to = qo * T + o;
            if (lane == 0 && to < to_n && t < tr.tau1) {
                const float s = inv[tr.kglob + t];
                gW[P.cumW[l] + (int64_t)to * tff + tr.toff + t] = make_float2(sx * s, sy * s);
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------
// input gradient.  Block = (fragment lt, one tile of its channels, sample group, part) and owns that part's
// contribution to those elements of gF.  It walks its share of the fragment's entries (triple, role, tile of the
// other operand); per entry the whole block
//   stages   the other operand's tile, the CG band and conj(W)/std of the tile in shared memory,
//   phase 1  builds the gFF tile  H[m][t1, t2] = sum_to conj(W[to, k])/std_k * gO[to, m]  for a chunk of m (warps
//            split m) and parks it in shared memory,
//   phase 2  lets every warp own rows m_t of the fragment and gather, in registers,
//            x[a] = sum C * conj(other[c][.]) * H[m][a, c]  over the band, adding x once to the block's accumulator.
// This is CGNet/cudaCG/cudaCG_FNWMM.cu:169-211 followed by cudaCG_sparse.cu:231-289 with gFF living only as one tile
// in shared memory.  Every sum has a fixed order; parts are added by parts_reduce_kernel in part order.
// ---------------------------------------------------------------------------------------------------------------

// phase 1 unit: H[m][K0 .. K0+KN) = sum_to wt[to][k] * gO[to, m]
template <int T, int NH, int NHP, int K0, int KN>
__device__ __forceinline__ void gf_h_unit(const float2* __restrict__ go, const float2* __restrict__ wt, float2* __restrict__ h,
                                          int to_n, int n, int mi) {
    static_assert(K0 % 2 == 0, "16-byte loads of the staged weights need an even first entry");
    float2 gt[KN];
#pragma unroll
    for (int k = 0; k < KN; ++k) gt[k] = make_float2(0.f, 0.f);
    // one output tile (T channels, adjacent in the slab) per step: its T loads are issued together, so their
    // global-load latencies overlap, and their offsets are compile-time constants
    for (int to0 = 0; to0 < to_n; to0 += T) {
        const float2* gp = go + ((to0 / T) * n + mi) * T * 32;
        float2 gvs[T];
#pragma unroll
        for (int j = 0; j < T; ++j) gvs[j] = to0 + j < to_n ? gp[j * 32] : make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < T; ++j) {
            if (to0 + j < to_n) {   // warp-uniform
                const float2 gv = gvs[j];
                const float4* w4 = reinterpret_cast<const float4*>(wt + (to0 + j) * NHP + K0);
#pragma unroll
                for (int k = 0; k < KN / 2; ++k) {
                    const float4 w = w4[k];
                    cfma(gt[2 * k], make_float2(w.x, w.y), gv);
                    cfma(gt[2 * k + 1], make_float2(w.z, w.w), gv);
                }
                if constexpr (KN % 2 == 1) cfma(gt[KN - 1], wt[(to0 + j) * NHP + K0 + KN - 1], gv);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < KN; ++k) h[(K0 + k) * 32] = gt[k];
}

// PRE: the gFF tiles were computed beforehand by the tensor-core GEMM (gff_tc.cu) and sit in the workspace `gff` in the
// layout of H; phase 1 is then an asynchronous copy of the entry's tile - whole, with the next entry's staging under way
// (`nbuf` 2), or in chunks of Mc rows with one staging buffer (`nbuf` 1), which lets two blocks share an SM or a tile be
// larger than the buffer.
//
// SHORTG (with `last_rep` > 1): the last sample group holds at most 32 / last_rep samples.  In that group a lane is a
// (row offset j, sample s) pair, s = lane % (32 / last_rep): a phase-1 unit covers last_rep rows m of the tile and a
// phase-2 unit last_rep rows of the owned fragment, one per lane group, instead of every lane repeating one row for an
// empty sample slot, so the group costs about 1 / last_rep of a full one.  Every element is still computed by one lane
// in the same order of operations: the bits do not change.
template <int T, bool DW, bool SPLIT, bool PRE = false, bool SHORTG = false>
__global__ void __launch_bounds__(kGfWarps * kWarp)
fused_gf_kernel(PlanDev P, const GfInfo* __restrict__ entries, const int* __restrict__ entry_begin,
                const int* __restrict__ blocks, const unsigned char* __restrict__ owner_tab, const float2* __restrict__ SF,
                const float2* __restrict__ SG, const float2* __restrict__ W, const float* __restrict__ inv,
                float2* __restrict__ out, int64_t part_stride, int B, int Mc, int max_n, int max_to, int band_floats,
                const float2* __restrict__ gff = nullptr, int64_t gff_stride = 0, const int64_t* __restrict__ gff_off = nullptr,
                int last_rep = 1, int nbuf = 2) {
    static_assert(!(SHORTG && SPLIT), "lane sharing of the short last group is written for whole-row units");
    using S = GfShape<T, DW>;
    constexpr int NH = S::NH, NHP = S::NHP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // blockIdx.x = block * G + group: the blocks are listed most expensive first, and the sample groups of one block
    // start together, so the cheap blocks of every group are what is left for the last wave
    const int G = (B + 31) >> 5;
    int blk = blockIdx.x / G, g = blockIdx.x - blk * G;
    if (SHORTG && last_rep > 1 && G > 1) {   // the cheap blocks of the short last group come after all others
        const int n_full = (int)(gridDim.x / G) * (G - 1);
        if ((int)blockIdx.x < n_full) {
            blk = blockIdx.x / (G - 1);
            g = blockIdx.x - blk * (G - 1);
        } else {
            blk = blockIdx.x - n_full;
            g = G - 1;
        }
    }
    const int lt = blocks[4 * blk], q = blocks[4 * blk + 1];
    const int part = blocks[4 * blk + 2], parts = blocks[4 * blk + 3];
    const int nt = 2 * lt + 1, t_0 = q * T;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int tau_t = P.tF[lt];
    float2* acc = reinterpret_cast<float2*>(smem_raw);          // [T][nt][32]
    float2* fo2 = acc + (size_t)T * max_n * 32;                  // 2 x [n_o][T][32]  other operand's tile, two entries
    float2* wt = fo2 + (size_t)nbuf * T * max_n * 32;            // [to_n][NHP]   conj(W) / std
    float* band2 = reinterpret_cast<float*>(wt + (size_t)max_to * NHP);   // 2 x [n][n2]
    unsigned short* ulist = reinterpret_cast<unsigned short*>(band2 + nbuf * band_floats);   // [warps][2 max_n] phase-2 units of each warp
    float2* H = reinterpret_cast<float2*>(reinterpret_cast<unsigned char*>(ulist) + ((kGfWarps * 4 * max_n + 15) & ~15));   // [Mc][NH][32]
    for (int i = threadIdx.x; i < T * nt * 32; i += blockDim.x) acc[i] = make_float2(0.f, 0.f);
    int n_units = 0;   // this warp's phase-2 units, listed once per block (every lane keeps the same count)
    for (int u = 0; u < gf_phase2_units<T, DW, SPLIT>(nt); ++u)
        if (owner_tab[2 * lt * lt + u] == warp) {
            if (lane == 0) ulist[warp * 2 * max_n + n_units] = (unsigned short)u;
            ++n_units;
        }
    __syncwarp();
    const float2* slabF = SF + (int64_t)g * P.nSF * 32;
    const float2* slabG = SG + (int64_t)g * P.nSO * 32 + lane;
    const bool shortg = SHORTG && last_rep > 1 && g == G - 1;   // block-uniform
    const int sh_w = 32 / (shortg ? last_rep : 1);              // sample slots in use
    const int sh_j = lane / sh_w, sh_s = lane - sh_j * sh_w;    // this lane's row offset inside a unit and its sample slot
    // phase 2 of one entry over the chunk of H that is resident
    auto gather = [&](bool first, const float2* fo, const float* band, int l, int lo_, int l2, int n2, int mc0, int mcn) {
        if (shortg) {   // (a constant false without SHORTG)  a unit = last_rep rows of the fragment, one per lane group
            for (int ug = warp; ug * last_rep < nt; ug += nwarps) {
                const int r = ug * last_rep + sh_j;
                if (r < nt) gf_phase2_unit<T, DW, false>(r, first, H, fo, band, acc, lt, nt, l, lo_, l2, n2, mc0, mcn, sh_s);
            }
            return;
        }
        for (int k = 0; k < n_units; ++k) {
            const int u = ulist[warp * 2 * max_n + k];
            gf_phase2_unit<T, DW, SPLIT>(u, first, H, fo, band, acc, lt, nt, l, lo_, l2, n2, mc0, mcn, lane);
        }
    };

    // Staging of an entry runs one entry ahead of its use: the other operand's tile and the CG band go to the idle
    // half of their double buffers by asynchronous copies issued when the previous entry starts; the tile of
    // conj(W)/std is fetched into registers before the previous entry's phase 2 (which does not read `wt`) and stored
    // after it.  No warp then waits at a barrier for another warp's global loads.
    auto stage_async = [&](const GfInfo& x, int buf) {
        const bool fst = x.role == 0;
        const int xn = 2 * x.l + 1, xn2 = 2 * x.l2 + 1, xno = fst ? xn2 : 2 * x.l1 + 1;
        const float4* src = reinterpret_cast<const float4*>(slabF + ((int64_t)x.fo_off + (DW ? q * xno * T : 0)) * 32);
        float4* dstf = reinterpret_cast<float4*>(fo2 + (size_t)buf * T * max_n * 32);
        for (int i = threadIdx.x; i < xno * T * 16; i += blockDim.x) __pipeline_memcpy_async(dstf + i, src + i, 16);
        float* dstb = band2 + buf * band_floats;
        for (int i = threadIdx.x; i < xn * xn2; i += blockDim.x) __pipeline_memcpy_async(dstb + i, P.cg + x.cgoff + i, 4);
        __pipeline_commit();
    };
    constexpr int kWtRegs = 2;   // staged weights a thread carries in registers across phase 2
    auto wt_load = [&](const GfInfo& x, int i) -> float2 {
        const bool fst = x.role == 0;
        const int xin0 = DW ? 0 : x.in0;
        const int t = i / NH, idx = i - t * NH;
        const int i1 = DW ? idx : idx / T, j1 = DW ? idx : idx % T;
        const int a = fst ? i1 : j1, c = fst ? j1 : i1;   // owned / other channel inside their tiles
        const bool ok = (t_0 + a < tau_t) && (DW || xin0 + c < x.tau_o);
        const int t1 = fst ? t_0 + a : xin0 + c, t2 = fst ? xin0 + c : t_0 + a;
        const int ch = DW ? t_0 + a : t1 * x.tau2 + t2;
        float2 w = make_float2(0.f, 0.f);
        if (ok) {
            w = __ldg(W + x.woff + (int64_t)t * x.tff + ch);
            const float sc = __ldg(inv + x.kglob + ch);
            w = make_float2(w.x * sc, -w.y * sc);
        }
        return w;
    };
    auto wt_prefetch = [&](const GfInfo& x, float2 (&reg)[kWtRegs]) {
#pragma unroll
        for (int j = 0; j < kWtRegs; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < x.to_n * NH) reg[j] = wt_load(x, i);
        }
    };
    auto wt_store = [&](const GfInfo& x, const float2 (&reg)[kWtRegs]) {
#pragma unroll
        for (int j = 0; j < kWtRegs; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < x.to_n * NH) wt[(i / NH) * NHP + i % NH] = reg[j];
        }
        for (int i = threadIdx.x + kWtRegs * blockDim.x; i < x.to_n * NH; i += blockDim.x)   // beyond the registers
            wt[(i / NH) * NHP + i % NH] = wt_load(x, i);
    };

    const int e_end = entry_begin[lt + 1];
    int e = entry_begin[lt] + part;
    GfInfo en;
    float2 wreg[kWtRegs];
    int buf = 0;
    if (e < e_end) {
        en = entries[e];
        if (!PRE || nbuf == 2) stage_async(en, 0);
        if constexpr (!PRE) wt_prefetch(en, wreg);
    }
    if constexpr (PRE) {
        if (nbuf == 1) {
            // Two blocks per SM: one staging buffer and the tile in chunks of Mc rows; while this block waits for its
            // copies the SM's other block computes.
            while (e < e_end) {
                const int l = en.l, n = 2 * l + 1, n2 = 2 * en.l2 + 1;
                const bool first = en.role == 0;
                GfInfo nx2 = en;
                if (e + parts < e_end) nx2 = entries[e + parts];
                if (en.to_n > 0) {
                    const int nt2 = (en.tau2 + T - 1) / T;
                    const int cell = en.cell0 + (first ? q * nt2 + en.in0 / T : (en.in0 / T) * nt2 + q);
                    const int64_t hoff = gff_off[l] + (int64_t)(cell - P.cell_begin[l]) * n * NH;
                    const float4* src = reinterpret_cast<const float4*>(gff + ((int64_t)g * gff_stride + hoff) * 32);
                    const int lo_ = first ? en.l2 : en.l1;
                    for (int mc0 = 0; mc0 < n; mc0 += Mc) {
                        const int mcn = min(Mc, n - mc0);
                        __syncthreads();   // the gather before this one is over: H (and for a new entry the staging buffer) is free
                        if (mc0 == 0) stage_async(en, 0);
                        float4* dst = reinterpret_cast<float4*>(H);
                        const float4* sc = src + (size_t)mc0 * NH * 16;
                        for (int i = threadIdx.x; i < mcn * NH * 16; i += blockDim.x) __pipeline_memcpy_async(dst + i, sc + i, 16);
                        __pipeline_commit();
                        __pipeline_wait_prior(0);
                        __syncthreads();
                        gather(first, fo2, band2, l, lo_, en.l2, n2, mc0, mcn);
                    }
                }
                en = nx2;
                e += parts;
            }
        }
        // The tiles come from the workspace: per entry one asynchronous copy of its tile into H, then the gather.  (Tried:
        // H as two half buffers with the next chunk's copy under way during the gather - the chunked gather cost more
        // than the hidden copy saved, 3.04 against 2.91 ms at lmax 14 with 16 channels.)
        GfInfo nxt;
        while (e < e_end) {
            const int l = en.l, n = 2 * l + 1, n2 = 2 * en.l2 + 1;
            const bool has_next = e + parts < e_end;
            const bool first = en.role == 0;
            if (has_next) nxt = entries[e + parts];
            __syncthreads();             // the previous entry's gather is over: H and the idle staging halves are free
            const bool live = en.to_n > 0;   // a degree without output channels has no tiles and contributes nothing
            if (live) {
                const int nt2 = (en.tau2 + T - 1) / T;
                const int cell = en.cell0 + (first ? q * nt2 + en.in0 / T : (en.in0 / T) * nt2 + q);
                const int64_t hoff = gff_off[l] + (int64_t)(cell - P.cell_begin[l]) * n * NH;
                const float4* src = reinterpret_cast<const float4*>(gff + ((int64_t)g * gff_stride + hoff) * 32);
                float4* dst = reinterpret_cast<float4*>(H);
                for (int i = threadIdx.x; i < n * NH * 16; i += blockDim.x) __pipeline_memcpy_async(dst + i, src + i, 16);
                __pipeline_commit();
            }
            if (has_next) {
                stage_async(nxt, buf ^ 1);
                __pipeline_wait_prior(1);   // the tile and this entry's staging have landed; the next entry's may still fly
            } else {
                __pipeline_wait_prior(0);
            }
            __syncthreads();
            const float2* fo = fo2 + (size_t)buf * T * max_n * 32;
            const float* band = band2 + buf * band_floats;
            const int lo_ = first ? en.l2 : en.l1;
            if (live) gather(first, fo, band, l, lo_, en.l2, n2, 0, n);
            en = nxt;
            e += parts;
            buf ^= 1;
        }
    }
    while (!PRE && e < e_end) {
        const bool has_next = e + parts < e_end;
        GfInfo nxt;
        if (has_next) nxt = entries[e + parts];
        const int l = en.l, n = 2 * l + 1, n2 = 2 * en.l2 + 1;
        const int to_n = en.to_n;
        const bool first = en.role == 0;   // the owned fragment is the first operand of this triple
        const float2* fo = fo2 + (size_t)buf * T * max_n * 32;
        const float* band = band2 + buf * band_floats;
        const int lo_ = first ? en.l2 : en.l1;
        wt_store(en, wreg);          // phase 1 of the previous entry ended before its second barrier
        __pipeline_wait_prior(0);    // this thread's copies for this entry have landed
        __syncthreads();             // staging visible; the previous entry's phase 2 is over: H and the other halves are free
        if (has_next) stage_async(nxt, buf ^ 1);
        const float2* go = slabG + (int64_t)en.go_off * 32;
        for (int mc0 = 0; mc0 < n; mc0 += Mc) {
            const int mcn = min(Mc, n - mc0);
            if (mc0 > 0) __syncthreads();   // the previous chunk's readers are done with H
            if (shortg) {   // (a constant false without SHORTG)  a unit = last_rep rows of the chunk, one per lane group
                const float2* gos = go - lane + sh_s;
                if constexpr (S::KA > 0) {
                    for (int u = warp; (u >> 1) * last_rep < mcn; u += nwarps) {
                        const int mi = mc0 + (u >> 1) * last_rep + sh_j;
                        if (mi < mc0 + mcn) {
                            float2* h = H + (size_t)(mi - mc0) * NH * 32 + sh_s;
                            if (u & 1) gf_h_unit<T, NH, NHP, S::KA, NH - S::KA>(gos, wt, h, to_n, n, mi);
                            else gf_h_unit<T, NH, NHP, 0, S::KA>(gos, wt, h, to_n, n, mi);
                        }
                    }
                } else {
                    for (int u = warp; u * last_rep < mcn; u += nwarps) {
                        const int mi = mc0 + u * last_rep + sh_j;
                        if (mi < mc0 + mcn) gf_h_unit<T, NH, NHP, 0, NH>(gos, wt, H + (size_t)(mi - mc0) * NH * 32 + sh_s, to_n, n, mi);
                    }
                }
            } else if constexpr (S::KA > 0) {
                for (int u = warp; u < 2 * mcn; u += nwarps) {
                    const int mi = mc0 + (u >> 1);
                    float2* h = H + (size_t)(mi - mc0) * NH * 32 + lane;
                    if (u & 1) gf_h_unit<T, NH, NHP, S::KA, NH - S::KA>(go, wt, h, to_n, n, mi);
                    else gf_h_unit<T, NH, NHP, 0, S::KA>(go, wt, h, to_n, n, mi);
                }
            } else {
                for (int mi = mc0 + warp; mi < mc0 + mcn; mi += nwarps)
                    gf_h_unit<T, NH, NHP, 0, NH>(go, wt, H + (size_t)(mi - mc0) * NH * 32 + lane, to_n, n, mi);
            }
            __syncthreads();
            if (has_next && mc0 + Mc >= n) wt_prefetch(nxt, wreg);   // in flight during the last chunk's phase 2
            gather(first, fo, band, l, lo_, en.l2, n2, mc0, mcn);
        }
        en = nxt;
        e += parts;
        buf ^= 1;
    }
    __syncthreads();
    float2* dst = out + (int64_t)part * part_stride;
    for (int i = threadIdx.x; i < T * nt * 32; i += blockDim.x) {
        const int ln = i & 31, rest = i >> 5;
        const int a = rest / nt, r = rest - a * nt;
        const int b = g * 32 + ln;
        if (b < B && t_0 + a < tau_t) dst[(int64_t)b * P.n_F + P.cumF[lt] + (int64_t)(t_0 + a) * nt + r] = acc[i];
    }
}

// out[b][e] = sum over the parts of e's fragment, in part order (partial: [part][B][n_total]).  With skip_single the
// fragments that were not split are left alone: their only part was written to `out` directly.
__global__ void __launch_bounds__(256)
parts_reduce_kernel(const int64_t* __restrict__ cum, int n_deg, int64_t n_total, const int* __restrict__ parts,
                    const float2* __restrict__ partial, int64_t part_stride, float2* __restrict__ out, int B, int skip_single) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_total) return;
    const int np = parts[find_degree(cum, n_deg, e)];
    if (skip_single && np <= 1) return;
    for (int b = blockIdx.y; b < B; b += gridDim.y) {
        const float2* src = partial + (int64_t)b * n_total + e;
        float2 s = src[0];
        for (int k = 1; k < np; ++k) {
            const float2 v = src[(int64_t)k * part_stride];
            s.x += v.x;
            s.y += v.y;
        }
        out[(int64_t)b * n_total + e] = s;
    }
}

void launch_parts_reduce(int kid, const int64_t* cum, int n_deg, int64_t n_total, const int* parts, const float2* partial,
                         int64_t part_stride, float2* out, int B, bool skip_single, cudaStream_t st) {
    if (n_total <= 0 || B <= 0) return;
    const unsigned gx = (unsigned)((n_total + 255) / 256);
    launch_begin(kid, st);
    parts_reduce_kernel<<<dim3(gx, (unsigned)std::min<int64_t>(B, 65535)), 256, 0, st>>>(cum, n_deg, n_total, parts, partial, part_stride,
                                                                                       out, B, skip_single ? 1 : 0);
    launch_end(kid, st);
}

}  // namespace cgb200

using namespace cgb200;

namespace {

struct Workspace {
    float2* SF;
    float2* SG;     // slab of gO in the backward
    float* inv;
    int* counters;  // one row counter per sample group
    float2* gf_part; // partial input gradients, [parts][B][n_F], when the input-gradient blocks are split
    int gf_level;
    float* tc_pack;  // packed TF32 weights of the tensor-core forward
    float2* fwd_part; // partial outputs, [parts][B][n_O], when the tensor-core forward splits its contraction
    int fwd_level;
    float2* gw_part; // partial weight gradients, [slices][w_len], when the sample groups are split over warps
    int gw_slices;
    float2* ff;      // forward with a statistics update: the generated tiles, written by the statistics kernel and read
                     // back by the tensor-core forward (same layout as gff); null when not used
    float* gff_pack; // packed conj(W)/std of the mid-gradient GEMM
    float2* gff;     // its output: the gFF tiles of every cell, [group][cell][m][tile entry][32 lanes]
    int gff_level;
    int64_t bytes;
};

// Slices of the sample groups in the weight-gradient kernel: a task walks all groups of its slice in sequence, so with
// few tasks the longest one sets the kernel's duration; slicing shortens it and multiplies the number of warps.
int gw_slices(const cgb200_plan* p, int64_t G) {
    if (p->d.depthwise) return 1;
    const int64_t n_tasks = p->gw_begin.empty() ? 0 : p->gw_begin.back();
    if (n_tasks == 0) return 1;
    int64_t s = (24 * (int64_t)p->num_sms + n_tasks - 1) / n_tasks;
    s = std::min<int64_t>(s, G);
    while (s > 1 && s * p->d.w_len * (int64_t)sizeof(float2) > (256ll << 20)) --s;
    return (int)std::max<int64_t>(s, 1);
}

// Phase-2 units of the input-gradient kernel: whole rows (default, faster at every shape measured) or rows split into
// two channel groups (CGB200_OPT_GRAD_F_SPLIT).  The plan holds a warp assignment for both.
bool gf_split(const cgb200_plan* p) { return p->opt[CGB200_OPT_GRAD_F_SPLIT] == 1; }

// Splitting level of the input-gradient kernel.  One block owns an SM (221 KB of shared memory) and the blocks differ
// widely in length, so with few blocks per SM the longest ones set the kernel's duration (measured with clock64 at lmax
// 14 with 16 channels and two blocks per SM: the SMs were busy with blocks 65 % of the time), while a block also has a
// fixed cost (accumulator set-up, write-out, one more partial sum to add) that makes very short blocks a loss (the
// 5-channel benchmark layer got 7 % slower one level further down).  The plan models a block's cost as its complex
// multiply-adds per lane - measured at three shapes: about 1050 units per microsecond - and the launch takes the coarsest
// level whose longest block is under a tenth of the ideal per-SM time, or under about 80 us.  Against the former
// "two blocks per SM": backward of the lmax-14 16-channel layer 8.5 -> 6.4 ms, lmax 10 with 32 channels 12.5 -> 10.0 ms.
int gf_level(const cgb200_plan* p, int64_t G) {
    const double ideal = p->gf_total_cost * (double)G / std::max(p->num_sms, 1);
    const double limit = std::max(0.1 * ideal, 85000.0);
    for (int lv = 0; lv < cgb200_plan::kGfLevels; ++lv)
        if (p->gf2_longest[lv] <= limit) return lv;
    return cgb200_plan::kGfLevels - 1;
}

int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

// How many lane groups share the last sample group's work when it is at most half full (1: none).  The CUDA-core weight
// gradient, whose per-lane results are summed over the whole warp anyway, lets the idle lanes take a share of its outer
// loop; the input gradient gives each lane group another row of a unit.  CGB200_OPT_SHORT_GROUP 0 switches it off.
int last_group_rep(const cgb200_plan* p, int64_t B, int64_t G) {
    if (p->opt[CGB200_OPT_SHORT_GROUP] == 0) return 1;
    const int64_t rem = B - 32 * (G - 1);
    return rem <= 4 ? 8 : rem <= 8 ? 4 : rem <= 16 ? 2 : 1;
}

// Shared memory of the input-gradient kernel: the part that does not depend on how many rows of a gFF tile H holds, and
// the bytes per row.
void gf_smem(const cgb200_plan* p, size_t* fixed, size_t* per_m) {
    const int T = p->d.tile;
    const int NHh = p->d.depthwise ? T : T * T;
    const int max_to = std::max(p->max_tau_out, 1);
    *fixed = (size_t)3 * T * p->max_n * 32 * sizeof(float2) + (size_t)max_to * ((NHh + 1) & ~1) * sizeof(float2) +
             2 * p->gen_band_bytes + (size_t)((kGfWarps * 4 * p->max_n + 15) & ~15);
    *per_m = (size_t)NHh * 32 * sizeof(float2);
}

// Shared memory of the input-gradient kernel's gather form (tiles read back from the workspace) with one staging buffer
// and no staged weights, without the rows of the tile.
size_t gf_gather_fixed(const cgb200_plan* p) {
    return (size_t)2 * p->d.tile * p->max_n * 32 * sizeof(float2) + p->gen_band_bytes + (size_t)((kGfWarps * 4 * p->max_n + 15) & ~15);
}

// The mid activation's gradient by a tensor-core GEMM into the workspace (gff_tc.cu) instead of tile by tile inside the
// input-gradient kernel.  Needs the plan's tables (tile edge 4, full product), at least a third of an entry's tile in that
// kernel's shared memory, and 8 bytes of workspace per sample and element of the (tile-padded) mid activation - at most
// 16 GB by default.  On from 12 output channels (measured on B200, backward of one layer: lmax 14 with 16 channels and 64
// samples 4.84 -> 3.41 ms, lmax 10 with 32 channels 8.06 -> 3.92 ms, lmax 10 with 16 channels 1.51 -> 1.10 ms; the GEMM
// writes its output at 5.1 TB/s); CGB200_OPT_GRAD_MID_GEMM overrides.
bool gff_wanted(const cgb200_plan* p, int64_t G) {
    if (!p->gff_ok || p->d.depthwise || p->opt[CGB200_OPT_GRAD_F_SPLIT] == 1 || tc_gf_wanted(p)) return false;
    const int opt = p->opt[CGB200_OPT_GRAD_MID_GEMM];
    if (opt == 0) return false;
    size_t fixed = 0, per_m = 0;
    gf_smem(p, &fixed, &per_m);
    // the kernel that reads the tiles back holds a whole tile, or - with one staging buffer - a third of its rows or more
    if (fixed + (size_t)p->max_n * per_m > kMaxDynSmem && gf_gather_fixed(p) + (size_t)((p->max_n + 2) / 3) * per_m > kMaxDynSmem)
        return false;
    if (opt >= 1) return true;
    const double bytes = (double)gff_group_elems(p) * (double)G * 32 * sizeof(float2);
    return p->max_tau_out >= 12 && bytes <= 16.0 * (1ull << 30);
}

// Forward with a statistics update: the statistics kernel generates every tile of the mid activation anyway; it then
// also writes them to the workspace and the forward kernel loads its tile instead of generating it a second time (same
// bits: both run the same generator).  Full product; on the tensor-core path tile edge 4 (not the staged variants), on
// the CUDA-core path tile edges 4 and up (below that generating a tile costs less than fetching it); at most 16 GB;
// CGB200_OPT_FWD_KEEP_MID overrides.
bool ff_store_wanted(const cgb200_plan* p, int64_t G) {
    if (!p->tiles_ok || p->d.depthwise) return false;
    if (tc_wanted(p) && (p->d.tile != 4 || p->opt[CGB200_OPT_TC_STAGED] >= 1)) return false;
    const int opt = p->opt[CGB200_OPT_FWD_KEEP_MID];
    if (opt == 0) return false;
    if (opt == 1) return true;
    const double bytes = (double)gff_group_elems(p) * (double)G * 32 * sizeof(float2);
    return p->d.tile >= 4 && bytes <= 16.0 * (1ull << 30);
}

// Layout of the caller's workspace.  The forward needs only the input slab, the norm factors, the row counters and
// (tensor-core forward) the packed weights; the backward adds the slab of the output gradient and the partial sums.
// Both layouts start at the same base and nothing in the workspace survives a call, so a buffer sized for the larger
// one serves both.
// `mode`: the backward (which also covers everything a forward needs), a forward with a statistics update, or a forward
// without one (no room for kept tiles).
enum { kWsBwd = 0, kWsFwdTrain = 1, kWsFwdInfer = 2 };
Workspace carve(const cgb200_plan* p, int64_t B, void* base, int mode = kWsBwd) {
    const int64_t G = (B + 31) / 32;
    const bool fwd_only = mode != kWsBwd;
    Workspace w{};
    int64_t off = 0;
    char* c = (char*)base;
    // first, at the same place in the forward's and the backward's layout: the tiles a forward with a statistics update
    // keeps (a backward given the same workspace with CGB200_FN_KEEP_MID reads them)
    w.ff = nullptr;
    if (mode != kWsFwdInfer && ff_store_wanted(p, G)) {
        w.ff = (float2*)(c + off);
        off += align256(gff_group_elems(p) * G * 32 * (int64_t)sizeof(float2));
    }
    w.SF = (float2*)(c + off);
    off += align256(std::max<int64_t>(p->d.nSF, 1) * G * 32 * (int64_t)sizeof(float2));
    w.SG = (float2*)(c + off);
    if (!fwd_only) off += align256(std::max<int64_t>(p->d.nSO, 1) * G * 32 * (int64_t)sizeof(float2));
    w.inv = (float*)(c + off);
    off += align256(std::max<int64_t>(p->d.sum_tff, 1) * (int64_t)sizeof(float));
    w.counters = (int*)(c + off);
    off += align256(G * (int64_t)sizeof(int));
    w.gf_level = gf_level(p, G);
    w.gf_part = (float2*)(c + off);
    if (!fwd_only && p->gf2_max_parts[w.gf_level] > 1)
        off += align256((int64_t)p->gf2_max_parts[w.gf_level] * B * std::max<int64_t>(p->d.n_F, 1) * (int64_t)sizeof(float2));
    w.tc_pack = (float*)(c + off);
    if (tc_wanted(p)) off += align256(tc_pack_floats(p) * (int64_t)sizeof(float));
    w.fwd_level = tc_wanted(p) ? tc_fwd_level(p, G) : 0;
    w.fwd_part = (float2*)(c + off);
    if (tc_wanted(p) && p->tc_max_parts[w.fwd_level] > 1)
        off += align256((int64_t)p->tc_max_parts[w.fwd_level] * B * std::max<int64_t>(p->d.n_O, 1) * (int64_t)sizeof(float2));
    w.gw_slices = gw_slices(p, G);
    w.gw_part = (float2*)(c + off);
    if (!fwd_only && w.gw_slices > 1) off += align256((int64_t)w.gw_slices * p->d.w_len * (int64_t)sizeof(float2));
    w.gff_level = tc_fwd_level(p, G);
    w.gff_pack = (float*)(c + off);
    w.gff = nullptr;
    if (!fwd_only && gff_wanted(p, G)) {
        off += align256(gff_pack_floats(p) * (int64_t)sizeof(float));
        w.gff = (float2*)(c + off);
        off += align256(gff_group_elems(p) * G * 32 * (int64_t)sizeof(float2));
    }
    w.bytes = off;
    return w;
}

int check_layer(const cgb200_plan* p, int64_t B, const void* ws, int64_t ws_bytes, int mode) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    CGB_REQUIRE(p->d.has_out, "the plan was created without tau_out");
    CGB_REQUIRE(B >= 0 && B <= 65535 * 32, "batch size out of range (at most 2097120 samples per call of the fused layer)");
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    CGB_REQUIRE(dev == p->device, "the plan belongs to another CUDA device than the current one");
    if (B > 0) {
        const int64_t need = carve(p, B, nullptr, mode).bytes;
        if (ws == nullptr || ws_bytes < need) {
            set_error("workspace too small: need " + std::to_string(need) + " bytes");
            return CGB200_ERR_WORKSPACE;
        }
        CGB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255) == 0, "workspace must be 256-byte aligned");
    }
    return CGB200_OK;
}

bool al8(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; }

bool has_pad(const std::vector<int>& tau, int T) {
    for (int t : tau)
        if (t % T) return true;
    return false;
}

int launch_prep(const cgb200_plan* p, const PrepJob& a, const PrepJob& b, int njobs, int B, int G, const float* stds, float eps,
                float* inv, int* counters, cudaStream_t st) {
    const int64_t maxN = std::max(a.N, njobs > 1 ? b.N : 0);
    const int gx = (int)std::min<int64_t>((maxN + 31) / 32, 2048);
    launch_begin(K_PREP, st);
    prep_kernel<<<dim3(std::max(gx, 1), G, njobs), 256, 0, st>>>(a, b, p->d.lmax, p->d.tile, B, stds, eps, inv, p->d.sum_tff,
                                                              counters, G);
    launch_end(K_PREP, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // namespace

// Run a statement with NN bound to the forward kernels' output-channel width as a compile-time constant.
#define CGB_DISPATCH_NTO(N_, ...)                                         \
    switch (N_) {                                                         \
        case 4: { constexpr int NN = 4; __VA_ARGS__; break; }             \
        case 5: { constexpr int NN = 5; __VA_ARGS__; break; }             \
        case 8: { constexpr int NN = 8; __VA_ARGS__; break; }             \
        default: { constexpr int NN = 16; __VA_ARGS__; break; }           \
    }

template <int T>
struct GwShape {   // output channels per weight-gradient task; must match gw_to of the plan (kGwTo in plan.cu)
    static constexpr int TO = T == 1 ? 8 : T == 2 ? 8 : T == 3 ? 4 : T == 4 ? 4 : T == 5 ? 5 : 6;
};

extern "C" {

int64_t cgb200_layer_workspace_bytes(const cgb200_plan* p, int64_t B) {
    if (p == nullptr || B < 0) {
        set_error("null plan or negative batch");
        return -1;
    }
    return carve(p, std::max<int64_t>(B, 1), nullptr).bytes;
}

int cgb200_layer_keeps_mid(const cgb200_plan* p, int64_t B) {
    if (p == nullptr || B <= 0) return 0;
    // the reader in the backward is the tensor-core weight gradient at tile edge 4
    return ff_store_wanted(p, (B + 31) / 32) && p->d.tile == 4 && tc_gw_wanted(p) ? 1 : 0;
}

int64_t cgb200_layer_fwd_workspace_bytes_for(const cgb200_plan* p, int64_t B, int flags) {
    if (p == nullptr || B < 0) {
        set_error("null plan or negative batch");
        return -1;
    }
    const bool update = (flags & CGB200_FN_PRESENT) && (flags & CGB200_FN_UPDATE);
    return carve(p, std::max<int64_t>(B, 1), nullptr, update ? kWsFwdTrain : kWsFwdInfer).bytes;
}

int64_t cgb200_layer_fwd_workspace_bytes(const cgb200_plan* p, int64_t B) {
    if (p == nullptr || B < 0) {
        set_error("null plan or negative batch");
        return -1;
    }
    return carve(p, std::max<int64_t>(B, 1), nullptr, kWsFwdTrain).bytes;
}

int cgb200_layer_fwd(const cgb200_plan* p, const float* F, const float* W, float* stds, float cnt, float eps, int flags,
                     float* O, int64_t B, void* workspace, int64_t workspace_bytes, void* stream) {
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    const bool update = fn && (flags & CGB200_FN_UPDATE);
    // a forward with a statistics update keeps its tiles when the workspace has room for them (the size
    // cgb200_layer_fwd_workspace_bytes_for gives for these flags); with the smaller workspace of a forward without an update
    // it runs all the same and keeps nothing
    int ws_mode = kWsFwdInfer;
    if (update && B > 0 && p != nullptr && workspace != nullptr && workspace_bytes >= carve(p, B, nullptr, kWsFwdTrain).bytes)
        ws_mode = kWsFwdTrain;
    int rc = check_layer(p, B, workspace, workspace_bytes, ws_mode);
    if (rc) return rc;
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    if (B == 0 || p->d.n_O == 0) return CGB200_OK;
    CGB_REQUIRE(F != nullptr && O != nullptr && (W != nullptr || p->d.w_len == 0), "null buffer");
    CGB_REQUIRE(al8(F) && al8(W) && al8(O), "buffers must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int G = (int)((B + 31) / 32);
    Workspace ws = carve(p, B, workspace, ws_mode);
    const int T = p->d.tile;

    PrepJob jf{(const float2*)F, ws.SF, p->d.n_F, p->d.cumF, p->d.cumSF, p->d.tF, p->d.nSF, has_pad(p->tF, T) ? 1 : 0};
    PrepJob none{};
    if ((rc = launch_prep(p, jf, none, 1, (int)B, G, fn ? stds : nullptr, eps, update ? nullptr : ws.inv, ws.counters, st)))
        return rc;
    bool ff_stored = false;
    if (update && p->d.n_cells > 0) {
        const size_t band = p->gen_band_bytes;
        launch_begin(K_STATS, st);
        // tile edge 5 and 6 need ~200 registers for a whole tile (one block of 8 warps per SM): two blocks per cell, each
        // with half the tile's rows and under 128 registers, put two blocks on an SM
        const int split_opt = p->opt[CGB200_OPT_STATS_SPLIT];
        const bool split_rows = !p->d.depthwise && (split_opt >= 0 ? split_opt != 0 : T >= 5);
        CGB_DISPATCH_TILE(T, p->d.depthwise, {
            auto kern = split_rows ? fused_stats_kernel<TT, DD, true> : fused_stats_kernel<TT, DD, false>;
            if (band > 40 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)band));
            kern<<<p->d.n_cells * (split_rows ? 2 : 1), 256, band, st>>>(p->d, ws.SF, stds, ws.inv, cnt, eps, (int)B, G,
                                                                        ws.ff, gff_group_elems(p), p->d_gff_off);
        });
        ff_stored = ws.ff != nullptr;
        launch_end(K_STATS, st);
        CGB_CUDA(cudaGetLastError());
    }
    const int n_rows = (int)p->fwd_rows.size() / 2;
    if (n_rows == 0) return CGB200_OK;
    if (tc_wanted(p))
        return launch_fwd_tc(p, ws.fwd_level, ws.SF, (const float2*)W, ws.inv, ws.tc_pack, (float2*)O, ws.fwd_part, (int)B, G,
                             ff_stored ? ws.ff : nullptr, st);
    // persistent shared-memory variant when one group's slab (plus reduction buffer and staging areas) fits in an SM
    const int NVh = p->d.depthwise ? T : T * T;
    // output channels per pass: the smallest instantiated width that covers the widest degree (at most kFwdTo)
    const int want_to = std::min(kFwdTo, std::max(p->max_tau_out, 1));
    const int red_to = want_to <= 4 ? 4 : want_to == 5 ? 5 : want_to <= 8 ? 8 : 16;
    const int stage_bytes = fwd_stage_bytes(red_to, NVh, p->max_n);
    const size_t slab_bytes = (size_t)p->d.nSF * 32 * sizeof(float2);
    const size_t smem_slab = slab_bytes + (size_t)kSlabWarps * (red_to * 32 * sizeof(float2) + stage_bytes);
    const size_t smem_rows = (size_t)kFwdWarps * (red_to * 32 * sizeof(float2) + stage_bytes);
    // 227 KB per block less the kernels' few bytes of static shared memory
    const bool fits = smem_slab <= kMaxDynSmem && G <= p->num_sms;
    const bool use_slab = fits && p->opt[CGB200_OPT_FWD_SLAB] != 0;
    if (smem_rows > kMaxDynSmem) {
        set_error("lmax too large for the fused forward kernel");
        return CGB200_ERR_UNSUPPORTED;
    }
    launch_begin(K_FWD, st);
    if (use_slab) {
        const int per_group = std::max(1, std::min(n_rows, p->num_sms / G));
        CGB_DISPATCH_TILE(T, p->d.depthwise, CGB_DISPATCH_NTO(red_to, {
            auto kern = fused_fwd_slab_kernel<TT, DD, NN>;
            CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_slab));
            kern<<<dim3(per_group, G), kSlabWarps * kWarp, smem_slab, st>>>(p->d, p->d_fwd_rows, n_rows, ws.SF, (const float2*)W,
                                                                         ws.inv, (float2*)O, (int)B, ws.counters, stage_bytes,
                                                                         ff_stored ? ws.ff : nullptr, gff_group_elems(p), p->d_gff_off);
        }));
    } else {
        CGB_DISPATCH_TILE(T, p->d.depthwise, CGB_DISPATCH_NTO(red_to, {
            auto kern = fused_fwd_kernel<TT, DD, NN>;
            if (smem_rows > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows));
            kern<<<dim3(n_rows, G), kFwdWarps * kWarp, smem_rows, st>>>(p->d, p->d_fwd_rows, ws.SF, (const float2*)W, ws.inv, (float2*)O,
                                                                     (int)B, stage_bytes, ff_stored ? ws.ff : nullptr,
                                                                     gff_group_elems(p), p->d_gff_off);
        }));
    }
    launch_end(K_FWD, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

// ---- inference with weights packed once ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
inv_std_kernel(const float* __restrict__ stds, float eps, float* __restrict__ inv, int n) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < n) inv[k] = stds == nullptr ? 1.f : 1.f / fmaxf(eps, stds[k]);
}

int64_t cgb200_layer_packed_weights_bytes(const cgb200_plan* p) {
    if (p == nullptr) {
        set_error("plan is null");
        return -1;
    }
    if (!p->d.has_out || !tc_wanted(p) || p->opt[CGB200_OPT_TC_STAGED] >= 1) return 0;
    return align256(tc_pack_floats(p) * (int64_t)sizeof(float)) + align256(std::max<int64_t>(p->d.sum_tff, 1) * (int64_t)sizeof(float));
}

int cgb200_layer_pack_weights(const cgb200_plan* p, const float* W, const float* stds, float eps, int flags, void* packed,
                              int64_t packed_bytes, void* stream) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    const int64_t need = cgb200_layer_packed_weights_bytes(p);
    CGB_REQUIRE(need > 0, "this plan's forward does not use packed weights (cgb200_layer_packed_weights_bytes is 0)");
    CGB_REQUIRE(packed != nullptr && packed_bytes >= need && (reinterpret_cast<uintptr_t>(packed) & 255) == 0,
                "the buffer for the packed weights is null, too small or not 256-byte aligned");
    const bool fn = (flags & CGB200_FN_PRESENT) != 0;
    CGB_REQUIRE(!fn || stds != nullptr, "stds is null although CGB200_FN_PRESENT is set");
    CGB_REQUIRE(W != nullptr && al8(W), "W is null or not 8-byte aligned");
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    CGB_REQUIRE(dev == p->device, "the plan belongs to another CUDA device than the current one");
    cudaStream_t st = (cudaStream_t)stream;
    float* pack = (float*)packed;
    float* inv = (float*)((char*)packed + align256(tc_pack_floats(p) * (int64_t)sizeof(float)));
    launch_begin(K_PREP, st);
    inv_std_kernel<<<(p->d.sum_tff + 255) / 256 + 1, 256, 0, st>>>(fn ? stds : nullptr, eps, inv, p->d.sum_tff);
    launch_end(K_PREP, st);
    CGB_CUDA(cudaGetLastError());
    return launch_fwd_tc(p, 0, nullptr, (const float2*)W, inv, pack, nullptr, nullptr, 0, 0, nullptr, st);
}

int cgb200_layer_fwd_packed(const cgb200_plan* p, const float* F, const void* packed, float* O, int64_t B, void* workspace,
                            int64_t workspace_bytes, void* stream) {
    int rc = check_layer(p, B, workspace, workspace_bytes, kWsFwdInfer);
    if (rc) return rc;
    CGB_REQUIRE(cgb200_layer_packed_weights_bytes(p) > 0, "this plan's forward does not use packed weights");
    CGB_REQUIRE(packed != nullptr && (reinterpret_cast<uintptr_t>(packed) & 255) == 0, "packed weights are null or misaligned");
    if (B == 0 || p->d.n_O == 0) return CGB200_OK;
    CGB_REQUIRE(F != nullptr && O != nullptr && al8(F) && al8(O), "null or misaligned buffer");
    cudaStream_t st = (cudaStream_t)stream;
    const int G = (int)((B + 31) / 32);
    Workspace ws = carve(p, B, workspace, kWsFwdInfer);
    const int T = p->d.tile;
    PrepJob jf{(const float2*)F, ws.SF, p->d.n_F, p->d.cumF, p->d.cumSF, p->d.tF, p->d.nSF, has_pad(p->tF, T) ? 1 : 0};
    PrepJob none{};
    if ((rc = launch_prep(p, jf, none, 1, (int)B, G, nullptr, 0.f, ws.inv, ws.counters, st))) return rc;
    if (p->fwd_rows.empty()) return CGB200_OK;
    return launch_fwd_tc(p, ws.fwd_level, ws.SF, nullptr, nullptr, (float*)packed, (float2*)O, ws.fwd_part, (int)B, G, nullptr, st);
}

int cgb200_layer_bwd(const cgb200_plan* p, const float* F, const float* W, const float* stds, float eps, int flags,
                     const float* gO, float* gF, float* gW, int64_t B, void* workspace, int64_t workspace_bytes,
                     void* stream) {
    int rc = check_layer(p, B, workspace, workspace_bytes, kWsBwd);
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
    CGB_REQUIRE(F != nullptr && (gO != nullptr || p->d.n_O == 0), "null buffer");
    CGB_REQUIRE(p->d.w_len == 0 || (W != nullptr && gW != nullptr), "W or gW is null");
    const int G = (int)((B + 31) / 32);
    Workspace ws = carve(p, B, workspace);
    const int T = p->d.tile;

    PrepJob jf{(const float2*)F, ws.SF, p->d.n_F, p->d.cumF, p->d.cumSF, p->d.tF, p->d.nSF, has_pad(p->tF, T) ? 1 : 0};
    PrepJob jg{(const float2*)gO, ws.SG, p->d.n_O, p->d.cumO, p->d.cumSO, p->d.tO, p->d.nSO, has_pad(p->tO, T) ? 1 : 0};
    if ((rc = launch_prep(p, jf, jg, p->d.n_O > 0 ? 2 : 1, (int)B, G, fn ? stds : nullptr, eps, ws.inv, ws.counters, st))) return rc;

    // The weight gradient and the input gradient are independent given gO.  Each leaves SMs idle towards its end
    // (few long blocks), so the weight gradient goes to a second stream forked from the caller's: its blocks fill the
    // SMs that the input gradient's last wave leaves free.  With per-kernel timing on, or when only one of the two
    // runs, everything stays on the caller's stream.
    const bool want_gf = p->d.n_F > 0 && gF != nullptr;
    // weight gradient (enqueued on stream gs): every (to, k) of every degree with both output and mid channels belongs to exactly one task
    const int n_tasks = p->gw_begin.empty() ? 0 : p->gw_begin.back();
    auto enqueue_gw = [&](cudaStream_t gs) -> int {
        if (tc_gw_wanted(p))
            return launch_gw_tc(p, ws.SF, ws.SG, ws.inv, (float2*)gW, ws.gw_part, ws.gw_slices, G,
                                (flags & CGB200_FN_KEEP_MID) ? ws.ff : nullptr, gs);
        const int blocks = (n_tasks + kGwWarps - 1) / kGwWarps;
        const int band_floats = (int)(p->gen_band_bytes / sizeof(float));
        const size_t smem = (size_t)kGwWarps * p->gen_band_bytes;
        if (smem > kMaxDynSmem) {
            set_error("lmax too large for the fused weight-gradient kernel");
            return CGB200_ERR_UNSUPPORTED;
        }
        launch_begin(K_GW, gs);
        if (p->d.depthwise) {
            CGB_DISPATCH_TILE(T, false, {
                auto kern = fused_gw_dw_kernel<TT>;
                if (smem > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                kern<<<blocks, kGwWarps * kWarp, smem, gs>>>(p->d, p->d_gw_tasks, n_tasks, ws.SF, ws.SG, ws.inv, (float2*)gW, G, band_floats);
            });
        } else {
            CGB_DISPATCH_TILE(T, false, {
                auto kern = fused_gw_kernel<TT, GwShape<TT>::TO>;
                if (smem > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                const int slices = ws.gw_slices;
                const int grid = (int)(((int64_t)n_tasks * slices + kGwWarps - 1) / kGwWarps);
                kern<<<grid, kGwWarps * kWarp, smem, gs>>>(p->d, p->d_gw_tasks, n_tasks, ws.SF, ws.SG, ws.inv,
                                                           slices > 1 ? ws.gw_part : (float2*)gW, G, band_floats, slices, p->d.w_len,
                                                           last_group_rep(p, B, G));
            });
            if (ws.gw_slices > 1) {
                launch_end(K_GW, gs);
                CGB_CUDA(cudaGetLastError());
                launch_gw_reduce(p, ws.gw_part, ws.gw_slices, (float2*)gW, gs);
                CGB_CUDA(cudaGetLastError());
                return CGB200_OK;
            }
        }
        launch_end(K_GW, gs);
        CGB_CUDA(cudaGetLastError());
        return CGB200_OK;
    };

    // input gradient (skipped when the caller passes no buffer: the first layer of a network needs none)
    auto enqueue_gf = [&]() -> int {
        const int lv = ws.gf_level;
        const int nblk = (int)p->gf2_blocks[lv].size() / 4;
        const bool split = p->gf2_max_parts[lv] > 1;
        const int64_t part_stride = split ? (int64_t)B * p->d.n_F : 0;
        float2* gf_out = split ? ws.gf_part : (float2*)gF;
        if (tc_gf_wanted(p)) {
            const int rc2 = launch_gf_tc(p, lv, ws.SF, ws.SG, (const float2*)W, ws.inv, gf_out, part_stride, (int)B, G, st);
            if (rc2) return rc2;
        } else {
            const int band_floats = (int)(p->gen_band_bytes / sizeof(float));
            const int max_to = std::max(p->max_tau_out, 1);
            const int last_rep = last_group_rep(p, B, G);   // lane sharing in a short last sample group
            size_t fixed = 0, per_m = 0;
            gf_smem(p, &fixed, &per_m);
            if (fixed + per_m > kMaxDynSmem) {
                set_error("lmax or tau_out too large for the fused input-gradient kernel");
                return CGB200_ERR_UNSUPPORTED;
            }
            const size_t budget = kMaxDynSmem;   // measured: one block of 16 warps with all m of an entry beats two half-size blocks
            const int Mc = (int)std::min<size_t>(p->max_n, (budget - fixed) / per_m);
            const size_t smem = fixed + (size_t)Mc * per_m;
            if (ws.gff != nullptr && T == 4 && !gf_split(p)) {
                int Mc_pre = Mc;
                size_t smem_pre = smem;
                int nbuf = 2, max_to_pre = max_to;
                const size_t fixed2 = gf_gather_fixed(p);
                if (Mc < p->max_n) {
                    // The whole tile does not fit beside two staging buffers (lmax 15 and more): one staging buffer and
                    // the tile in chunks, one block per SM.
                    nbuf = 1;
                    max_to_pre = 0;
                    Mc_pre = (int)std::min<size_t>(p->max_n, (kMaxDynSmem - fixed2) / per_m);
                    smem_pre = fixed2 + (size_t)Mc_pre * per_m;
                }
                // Two blocks per SM (the gather variant needs 64 registers per thread, so shared memory decides): one
                // staging buffer instead of two, no staged weights, and the tile in chunks of as many rows as half an
                // SM's shared memory leaves.  The SM's other block computes while a block waits for its copies, which
                // the single block could only hide for the small staging copies.  Measured at 64 samples: lmax 10 with
                // 16 channels 801 -> 709 us, with 32 channels 2892 -> 2582 us, lmax 14 with 16 channels (three chunks
                // per tile) 2816 -> 2767 us.  Taken when the launch has at least two blocks for every SM;
                // CGB200_OPT_GRAD_MID_GEMM 2 / 3 force it on / off.
                {
                    const size_t limit = (kSmemPerSM - 2 * 1024) / 2;   // two blocks, 1 KB reserved for each
                    const int mode = p->opt[CGB200_OPT_GRAD_MID_GEMM];
                    const bool fits = fixed2 + 4 * per_m <= limit;
                    const int Mc2 = fits ? (int)std::min<size_t>(p->max_n, (limit - fixed2) / per_m) : 0;
                    const bool pays = 3 * Mc2 >= p->max_n && (int64_t)nblk * G >= 2 * (int64_t)p->num_sms;   // at most three chunks
                    if (fits && mode != 3 && (mode == 2 || pays)) {
                        nbuf = 1;
                        max_to_pre = 0;
                        Mc_pre = Mc2;
                        smem_pre = fixed2 + (size_t)Mc_pre * per_m;
                    }
                }
                const int rc2 = launch_gff_tc(p, ws.gff_level, ws.SG, (const float2*)W, ws.inv, ws.gff_pack, ws.gff, G, st);
                if (rc2) return rc2;
                auto kern = last_rep > 1 ? fused_gf_kernel<4, false, false, true, true> : fused_gf_kernel<4, false, false, true, false>;
                if (smem_pre > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_pre));
                CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
                launch_begin(K_GF, st);
                kern<<<(unsigned)((int64_t)nblk * G), kGfWarps * kWarp, smem_pre, st>>>(
                    p->d, p->d_gf_info, p->d_gf_begin, p->d_gf2_blocks[lv], p->d_gf_owner, ws.SF, ws.SG, (const float2*)W, ws.inv, gf_out,
                    part_stride, (int)B, Mc_pre, p->max_n, max_to_pre, band_floats, ws.gff, gff_group_elems(p), p->d_gff_off, last_rep, nbuf);
                launch_end(K_GF, st);
                CGB_CUDA(cudaGetLastError());
            } else {
            launch_begin(K_GF, st);
            // phase-2 shape: whole rows, or the owned channels of a row split over two units (see gf_split)
            const bool split_units = gf_split(p);
            const unsigned char* owner = p->d_gf_owner + (size_t)(split_units ? 1 : 0) * 2 * (p->d.lmax + 1) * (p->d.lmax + 1);
            CGB_DISPATCH_TILE(T, p->d.depthwise, {
                auto kern = split_units ? fused_gf_kernel<TT, DD, true, false, false>
                                        : last_rep > 1 ? fused_gf_kernel<TT, DD, false, false, true> : fused_gf_kernel<TT, DD, false, false, false>;
                if (smem > 48 * 1024) CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                kern<<<(unsigned)((int64_t)nblk * G), kGfWarps * kWarp, smem, st>>>(p->d, p->d_gf_info, p->d_gf_begin, p->d_gf2_blocks[lv], owner, ws.SF, ws.SG, (const float2*)W, ws.inv, gf_out, part_stride, (int)B, Mc, p->max_n, max_to, band_floats, nullptr, 0, nullptr, split_units ? 1 : last_rep, 2);
            });
            launch_end(K_GF, st);
            CGB_CUDA(cudaGetLastError());
            }
        }
        if (split) {
            launch_parts_reduce(K_GF_REDUCE, p->d.cumF, p->d.lmax + 1, p->d.n_F, p->d_gf2_parts[lv], ws.gf_part, part_stride, (float2*)gF,
                                (int)B, false, st);
            CGB_CUDA(cudaGetLastError());
        }
        return CGB200_OK;
    };

    const bool want_gw = n_tasks > 0;
    if (!(want_gw && want_gf) || timing_active() || p->opt[CGB200_OPT_BWD_SERIAL] == 1) {
        if (want_gw && (rc = enqueue_gw(st))) return rc;
        if (want_gf && (rc = enqueue_gf())) return rc;
        return CGB200_OK;
    }
    std::lock_guard<std::mutex> side_lock(p->side_mutex);
    if (!p->side_stream) {
        CGB_CUDA(cudaStreamCreateWithFlags(&p->side_stream, cudaStreamNonBlocking));
        CGB_CUDA(cudaEventCreateWithFlags(&p->ev_fork, cudaEventDisableTiming));
        CGB_CUDA(cudaEventCreateWithFlags(&p->ev_join, cudaEventDisableTiming));
    }
    CGB_CUDA(cudaEventRecord(p->ev_fork, st));
    CGB_CUDA(cudaStreamWaitEvent(p->side_stream, p->ev_fork, 0));
    // from here on the join is enqueued whatever the launches return (a capturing stream must be joined)
    // the input gradient is enqueued first: its large blocks take the SMs, the weight gradient's small ones fill the tail
    const int rc_f = enqueue_gf();
    const int rc_w = enqueue_gw(p->side_stream);
    CGB_CUDA(cudaEventRecord(p->ev_join, p->side_stream));
    CGB_CUDA(cudaStreamWaitEvent(st, p->ev_join, 0));
    return rc_f ? rc_f : rc_w;
}

// ---------------------------------------------------------------------------------------------------------------
// Forward pass for callers that cannot allocate device memory.
//
// cgb200_layer_fwd takes its scratch (the rearranged activations, the per-channel norm factors and the row counters
// of the persistent forward kernel) from the caller.  Some hosts have no allocator to ask: a plugin entered from
// inside another framework's stream callback or graph-replay path, a process that handed all device memory to an
// arena it does not own, or an embedding where cudaMalloc is forbidden after start-up because it synchronises the
// device.  For them the scratch lives in the fixed array below, which every GPU that loads this library holds from
// module load until the process exits.
//
// The array's name is only a host-side handle: passing `g_static_scratch` itself to a kernel would hand it a host
// address.  Its device address is looked up once per device with cudaGetSymbolAddress, with that device current, on the
// first call made for that device; do that first call before starting any stream capture.
// ---------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[CGB200_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};   // device address of g_static_scratch, per device ordinal
}  // namespace

int cgb200_layer_fwd_static(const cgb200_plan* p, const float* F, const float* W, float* stds, float cnt, float eps,
                            int flags, float* O, int64_t B, void* stream) {
    CGB_REQUIRE(p != nullptr, "plan is null");
    CGB_REQUIRE(B >= 0, "negative batch size");
    const int64_t need = cgb200_layer_fwd_workspace_bytes_for(p, B, 0);   // the forward's own need without room for kept tiles
    if (need < 0) return CGB200_ERR_ARGUMENT;
    if (need > (int64_t)CGB200_STATIC_SCRATCH_BYTES) {
        set_error("cgb200_layer_fwd_static: the forward of this plan and batch needs " + std::to_string(need) +
                  " bytes of scratch, the built-in array holds " + std::to_string((int64_t)CGB200_STATIC_SCRATCH_BYTES) +
                  "; use a smaller batch or cgb200_layer_fwd with a caller-provided workspace");
        return CGB200_ERR_WORKSPACE;
    }
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    CGB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal out of range for the built-in scratch table");
    CGB_REQUIRE(dev == p->device, "the plan belongs to another CUDA device than the current one");
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        CGB_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        CGB_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address for the built-in scratch");
        g_static_scratch_ptr[dev] = ptr;
    }
    // Nothing in the array has to survive from one call to the next and nothing is assumed to be zero: the prep
    // kernel rewrites the slab (padding channels included), the norm factors and the row counters on every call.
    return cgb200_layer_fwd(p, F, W, stds, cnt, eps, flags, O, B, g_static_scratch_ptr[dev],
                            (int64_t)CGB200_STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
