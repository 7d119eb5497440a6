// Gradient of the quadratic mid activation as a tensor-core GEMM, for the input-gradient kernel to read back:
//
//   gFF_l[(m, b), (k, re|im)] = sum_to  gO_l[(m, b), (to, re|im)] * conj(W_l)[k, to] / std_k
//
// (CGNet/cudaCG/cudaCG_FNWMM.cu:169-211, the first half of the reference's backward.)  The fused input-gradient kernel
// builds this tile by tile on the CUDA cores and, because a cell's tile is needed by the blocks of both its operand
// fragments, twice; at 16 channels and more that is half of its time and more.  Here every tile is computed once, by
// tcgen05 MMAs, and written to a workspace in exactly the layout the input-gradient kernel keeps it in shared memory
// ([group of 32 samples][cell][m][tile entry][lane] complex), so that kernel's first phase becomes a copy.
//
// Block = one row tile (degree l, four consecutive m, one group of 32 samples: 128 rows = the 128 TMEM lanes) and a share
// of the degree's cells (the same tile lists and splitting levels as the tensor-core forward).  The A operand - the
// block's 128 rows of gO, (to, re|im) along K, split into TF32 high and low parts - is built once per block.  The cells
// are walked in groups that fill 32 KB of packed weights (4 cells at 16 output channels): `gff_pack_kernel` stores a
// group as one K-major matrix [high rows of its cells | low rows of its cells], so one MMA of width 64 nc computes Ah*Bh
// and Ah*Bl for all nc cells and a second of width 32 nc adds Al*Bh (3xTF32; a cell's contraction is only 2 tau_out long,
// so the accumulator needs no rounded partial sums).  Roles: warp 0 streams the groups' weights through a ring of three
// stages with bulk asynchronous copies, one lane of warp 1 issues the MMAs into two alternating accumulator regions,
// warps 2-5 read a finished region with tcgen05.ld, add the two halves and store the tiles (a warp owns the TMEM lanes of
// its m; each store instruction writes 256 contiguous bytes).  The kernel is bound by those stores: 8 bytes of HBM
// traffic per 2 tau_out complex multiply-adds.  Every wait is bounded as in the other tensor-core kernels.
#include <algorithm>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cgb200 {

constexpr int kGffStages = 3;
constexpr int kGffThreads = 32 * 6;
constexpr int kGffStageBytes = 32 * 1024;

// cells per group for a contraction of Kb floats: a group's packed weights, 64 rows per cell, fill at most one stage
__host__ __device__ inline int gff_group_cells(int Kb) { return Kb <= 32 ? 4 : Kb <= 64 ? 2 : 1; }
__host__ __device__ inline int gff_kb(int to_n) { return (2 * to_n + 7) & ~7; }

// ---------------------------------------------------------------------------------------------------------------
// Weight packing: one block per cell.  Row n' = 2 idx + (re|im) of the cell (idx = i T + j, the tile entry), column
// kk = 2 to + (re|im):  H.re = sum wr*gr - wi*gi,  H.im = sum wi*gr + wr*gi  with w = conj(W)/std.
// ---------------------------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256)
gff_pack_kernel(PlanDev P, const int64_t* __restrict__ pack_off, const float2* __restrict__ W, const float* __restrict__ inv,
                float* __restrict__ pack) {
    constexpr int NH = T * T;
    const int c = blockIdx.x;
    const CellInfo ci = P.cell_info[c];
    const int l = P.triples[P.cells[c].triple].l;
    const int to_n = P.tO[l];
    if (to_n == 0) return;
    const int Kb = gff_kb(to_n), CG = gff_group_cells(Kb);
    const int tff = P.tFF[l];
    const int k = c - P.cell_begin[l], ncell = P.cell_begin[l + 1] - P.cell_begin[l];
    const int gi = k / CG, cg = k - gi * CG, nc = min(CG, ncell - gi * CG);
    float* grp = pack + pack_off[l] + (int64_t)gi * CG * 64 * Kb;
    const float2* Wl = W + P.cumW[l];
    for (int e = threadIdx.x; e < NH * (Kb / 2); e += blockDim.x) {
        const int idx = e / (Kb / 2), to = e - idx * (Kb / 2);
        const int i = idx / T, j = idx - i * T;
        float2 w = make_float2(0.f, 0.f);
        if (to < to_n && i < ci.v1 && j < ci.v2) {
            const int ch = i * ci.tau2 + j;
            w = __ldg(Wl + (int64_t)to * tff + ci.wch0 + ch);
            const float sc = __ldg(inv + ci.kch0 + ch);
            w = make_float2(w.x * sc, -w.y * sc);
        }
        const float hr = to_tf32(w.x), hi = to_tf32(w.y);
        const int kk = 2 * to;
#pragma unroll
        for (int part = 0; part < 2; ++part) {   // high rows, then low rows
            const float vr = part ? w.x - hr : hr, vi = part ? w.y - hi : hi;
            const int r0 = part * nc * 32 + cg * 32 + 2 * idx, r1 = r0 + 1;
            const int o0 = (r0 >> 3) * (Kb / 4) * 32 + (kk >> 2) * 32 + (r0 & 7) * 4 + (kk & 3);
            const int o1 = (r1 >> 3) * (Kb / 4) * 32 + (kk >> 2) * 32 + (r1 & 7) * 4 + (kk & 3);
            *reinterpret_cast<float2*>(grp + o0) = make_float2(vr, -vi);
            *reinterpret_cast<float2*>(grp + o1) = make_float2(vi, vr);
        }
    }
}

template <int T>
__global__ void __launch_bounds__(kGffThreads)
gff_tc_kernel(PlanDev P, const int* __restrict__ tiles, const int64_t* __restrict__ pack_off, const int64_t* __restrict__ gff_off,
              const float2* __restrict__ SG, const float* __restrict__ pack, float2* __restrict__ gff, int64_t group_stride,
              int* __restrict__ status, uint32_t wait_limit, int idle_mma) {
    constexpr int NH = T * T;
    static_assert(NH == 16, "built for tile edge 4: a cell is 32 real accumulator columns");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kGffStages], empty_bar[kGffStages], acc_full[2], acc_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;

    const int l = tiles[4 * blockIdx.x], m0 = tiles[4 * blockIdx.x + 1];
    const int part = tiles[4 * blockIdx.x + 2], parts = tiles[4 * blockIdx.x + 3];
    const int g = blockIdx.y;
    const int n = 2 * l + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int to_n = P.tO[l];
    const int Kb = gff_kb(to_n), CG = gff_group_cells(Kb);
    const int ncell_deg = P.cell_begin[l + 1] - P.cell_begin[l];
    const int groups_deg = (ncell_deg + CG - 1) / CG;
    const int g0 = (int)((int64_t)groups_deg * part / parts), g1 = (int)((int64_t)groups_deg * (part + 1) / parts);
    const uint32_t sbo = (uint32_t)(Kb / 4) * 128;   // bytes between consecutive 8-row groups of a K-major operand
    const uint32_t a_bytes = 128u * (uint32_t)Kb * 4u;
    unsigned char* a_hi = smem_raw;
    unsigned char* a_lo = a_hi + a_bytes;
    unsigned char* ring = a_lo + a_bytes;
    const uint32_t region_cols = 64u * (uint32_t)CG;
    const uint32_t tmem_cols = 2 * region_cols <= 128 ? 128u : 2 * region_cols <= 256 ? 256u : 512u;
    volatile int* failed = &failed_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGffStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int r = 0; r < 2; ++r) {
            mbar_init(&acc_full[r], 1);
            mbar_init(&acc_free[r], 4);   // one arrival per store warp
        }
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    // A operand: row r = 32 (m - m0) + sample, columns (to, re|im); K-major core matrices of 8 rows x 16 bytes
    {
        const float2* slab = SG + ((int64_t)g * P.nSO + P.cumSO[l]) * 32;
        const int quads = Kb / 4;   // 16-byte pieces (two output channels) per row
        for (int e = threadIdx.x; e < 128 * quads; e += blockDim.x) {
            const int qd = e >> 7, r = e & 127;   // consecutive threads take consecutive rows: coalesced loads, conflict-free stores
            const int mi = m0 + (r >> 5), ln = r & 31;
            float2 x0 = make_float2(0.f, 0.f), x1 = x0;
            const int to = 2 * qd;
            if (mi < n) {
                if (to < to_n) x0 = slab[(((to / T) * n + mi) * T + to % T) * 32 + ln];
                if (to + 1 < to_n) x1 = slab[((((to + 1) / T) * n + mi) * T + (to + 1) % T) * 32 + ln];
            }
            float4 h, w;
            h.x = to_tf32(x0.x); h.y = to_tf32(x0.y); h.z = to_tf32(x1.x); h.w = to_tf32(x1.y);
            w.x = x0.x - h.x; w.y = x0.y - h.y; w.z = x1.x - h.z; w.w = x1.y - h.w;
            const size_t off = (size_t)(r >> 3) * sbo + (size_t)qd * 128 + (size_t)(r & 7) * 16;
            *reinterpret_cast<float4*>(a_hi + off) = h;
            *reinterpret_cast<float4*>(a_lo + off) = w;
        }
    }
    fence_proxy_async();   // the A operand becomes visible to the tensor core's async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const float* pack_l = pack + pack_off[l];
    const int n_groups = g1 - g0;

    if (warp == 0) {
        // ---------------- weights: one bulk copy per group ----------------
        bool ok = true;
        for (int j = 0; j < n_groups && ok; ++j) {
            const int s = j % kGffStages, u = j / kGffStages;
            if (u > 0) ok = mbar_wait_warp(&empty_bar[s], (uint32_t)((u - 1) & 1), failed, wait_limit);
            if (!ok) break;
            if (lane == 0) {
                const int gi = g0 + j;
                const int nc = min(CG, ncell_deg - gi * CG);
                const uint32_t bytes = (uint32_t)nc * 64u * (uint32_t)Kb * 4u;
                mbar_arrive_expect_tx(&full_bar[s], bytes);
                bulk_g2s(ring + (size_t)s * kGffStageBytes, pack_l + (int64_t)gi * CG * 64 * Kb, bytes, &full_bar[s]);
            }
        }
        // copies this warp started must have landed before the block gives up its shared memory
        if (lane == 0 && (!ok || *failed))
            for (int j = max(0, n_groups - kGffStages); j < n_groups; ++j)
                mbar_drain(&full_bar[j % kGffStages], (uint32_t)((j / kGffStages) & 1), wait_limit);
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && !idle_mma) {
            bool ok = true;
            const uint64_t dah0 = smem_desc(smem_u32(a_hi), 128, sbo), dal0 = smem_desc(smem_u32(a_lo), 128, sbo);
            for (int j = 0; j < n_groups && ok; ++j) {
                const int s = j % kGffStages, u = j / kGffStages, r = j & 1;
                const int nc = min(CG, ncell_deg - (g0 + j) * CG);
                if (j >= 2) ok = mbar_wait(&acc_free[r], (uint32_t)(((j >> 1) - 1) & 1), failed, wait_limit);
                if (!ok) break;
                ok = mbar_wait(&full_bar[s], (uint32_t)(u & 1), failed, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)r * region_cols;
                const uint64_t db0 = smem_desc(smem_u32(ring + (size_t)s * kGffStageBytes), 128, sbo);
                const uint32_t idesc_wide = tc_idesc(128, 64 * nc), idesc = tc_idesc(128, 32 * nc);
                for (int ks = 0; ks < Kb / 8; ++ks) {
                    const uint64_t dah = desc_advance(dah0, ks * 256), dal = desc_advance(dal0, ks * 256);
                    const uint64_t db = desc_advance(db0, ks * 256);
                    tc_mma_tf32(d, dah, db, idesc_wide, ks > 0 ? 1u : 0u);   // Ah x [Bh | Bl] -> columns 0 .. 64 nc
                    tc_mma_tf32(d, dal, db, idesc, 1u);                      // Al x Bh       -> columns 0 .. 32 nc
                }
                tc_commit(&empty_bar[s]);   // the stage's weights have been read
                tc_commit(&acc_full[r]);    // the group's tiles are complete
            }
        }
    } else {
        // ---------------- store warps ----------------
        const int wq = warp & 3;                      // the TMEM lane quarter this warp may read = its m inside the row tile
        const int mi = m0 + wq;
        const bool live_m = mi < n;
        float2* dst_l = gff + ((int64_t)g * group_stride + gff_off[l]) * 32 + lane;
        bool ok = true;
        for (int j = 0; j < n_groups && ok; ++j) {
            const int r = j & 1;
            const int gi = g0 + j;
            const int nc = min(CG, ncell_deg - gi * CG);
            ok = mbar_wait_warp(&acc_full[r], (uint32_t)((j >> 1) & 1), failed, wait_limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t base = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)r * region_cols;
            for (int c = 0; c < nc; ++c) {
                float2* dst = dst_l + ((int64_t)(gi * CG + c) * n + mi) * NH * 32;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t rh[16], rl[16];   // Ah Bh + Al Bh, and Ah Bl
                    tmem_ld16(base + (uint32_t)(c * 32 + half * 16), rh);
                    tmem_ld16(base + (uint32_t)(nc * 32 + c * 32 + half * 16), rl);
                    if (live_m) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            dst[(half * 8 + i) * 32] = make_float2(__uint_as_float(rh[2 * i]) + __uint_as_float(rl[2 * i]),
                                                                   __uint_as_float(rh[2 * i + 1]) + __uint_as_float(rl[2 * i + 1]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[r]);   // the region may be overwritten by group j + 2
        }
        if (!ok && live_m) {   // a block that gave up marks the tiles it owns
            const float nanv = __uint_as_float(kNaNBits);
            for (int gi = g0; gi < g1; ++gi)
                for (int c = 0; c < min(CG, ncell_deg - gi * CG); ++c)
                    for (int i = 0; i < NH; ++i) dst_l[(((int64_t)(gi * CG + c) * n + mi) * NH + i) * 32] = make_float2(nanv, nanv);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
int64_t gff_pack_floats(const cgb200_plan* p) { return p->gff_ok ? p->gff_pack_off.back() : 0; }
int64_t gff_group_elems(const cgb200_plan* p) { return p->tiles_ok ? p->gff_off.back() : 0; }

int launch_gff_tc(const cgb200_plan* p, int lv, const float2* SG, const float2* W, const float* inv, float* pack, float2* gff,
                  int G, cudaStream_t st) {
    if (!p->gff_ok || p->tc_tiles[lv].empty()) return CGB200_OK;
    launch_begin(K_GFF_PACK, st);
    if (p->d.n_cells > 0) gff_pack_kernel<4><<<p->d.n_cells, 256, 0, st>>>(p->d, p->d_gff_pack_off, W, inv, pack);
    launch_end(K_GFF_PACK, st);
    CGB_CUDA(cudaGetLastError());
    const int Kb = gff_kb(std::max(p->max_tau_out, 1));
    const size_t smem = (size_t)2 * 128 * Kb * 4 + (size_t)kGffStages * kGffStageBytes;
    auto kern = gff_tc_kernel<4>;
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int idle = p->opt[CGB200_OPT_TEST_IDLE_MMA] == 1 ? 1 : 0;
    launch_begin(K_GFF_GEMM, st);
    kern<<<dim3((unsigned)p->tc_tiles[lv].size() / 4, G), kGffThreads, smem, st>>>(p->d, p->d_tc_tiles[lv], p->d_gff_pack_off, p->d_gff_off,
                                                                                  SG, pack, gff, p->gff_off.back(), p->d_status,
                                                                                  wait_polls(p), idle);
    launch_end(K_GFF_GEMM, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // namespace cgb200
