// Tensor-core variant of the fused forward: CG product generated on the CUDA cores straight into shared memory as the
// A operand of a tcgen05 (5th-generation tensor core) GEMM whose accumulator lives in tensor memory; the mixing weights,
// pre-scaled by 1/std, split into TF32 high/low parts and packed in the MMA's shared-memory order, arrive by bulk
// asynchronous copy (the TMA engine's 1-D mode).  The quadratic mid activation FF exists only as one 128 x 2T^2 tile
// per pipeline stage.
//
//   O_l[(m, b), (to, re|im)] = sum_k  FF_l[(m, b), (k, re|im)] * Wr_l[(k, re|im), (to, re|im)]
//
// The complex product is run as a real GEMM of doubled dimensions: a row of A holds (re, im) of every mid channel, the
// columns of B hold, for output (to, re): (Wr, -Wi) and for (to, im): (Wi, Wr).  3xTF32: A = Ah + Al, B = Bh + Bl with
// Ah, Bh rounded to TF32; D = Ah*Bh + Al*Bh + Ah*Bl, accumulated in fp32 by the tensor core (the dropped Al*Bl term
// is ~2^-22 relative).  The packed weights hold Bl directly behind Bh, which makes [Bh | Bl] one K-major matrix of 2 N
// rows: one MMA of width 2 N computes Ah*Bh into accumulator columns 0 .. N and Ah*Bl into N .. 2 N, a second of width N
// adds Al*Bh - two instructions per K step instead of three (an MMA costs about 65 cycles to issue whatever its width,
// and each one re-reads its A tile from shared memory); the two column halves are added when the accumulator is read.
//
// Block = one row tile: degree l, four consecutive m, one group of 32 samples (row r = 32*(m - m0) + sample, the same
// one-sample-per-lane scheme as the other fused kernels, so the generator is gen_slab unchanged).  Warps:
//   generator groups 0..S-1 (S pipeline stages), four warps each: group s produces the cells k = s, s + S, ... of the
//     degree into pipeline stage s (A tile written with st.shared, then fence.proxy.async + mbarrier arrive); its first
//     lane also starts the bulk copy of the cell's packed weights into the stage;
//   one MMA warp: a single lane waits for each stage, issues the 3 x (2T^2/8) tcgen05.mma of the cell and commits them
//     to the stage's "empty" barrier;
//   flush warps (one or two groups of four): the tensor core adds into its fp32 accumulator with truncation, so the error
//     of a long contraction grows with the number of accumulation steps (measured 3e-3 at 180 k complex mid channels).
//     The cells are therefore summed in chunks of kChunkSteps accumulation steps into two alternating accumulator
//     regions; after each chunk a flush group reads the region with tcgen05.ld (a warp owns the TMEM lanes 32 (w % 4) ..
//     + 31 = its own m) and adds it to running sums in registers with ordinary rounded fp32 adds, then hands the region
//     back.  The flush warps write O at the end.
// Every wait is bounded: a wait that runs out sets a flag in shared memory and a status word in global memory, all
// roles then skip to the end, tensor memory is released and the kernel returns.
#include <cuda_pipeline.h>

#include <algorithm>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cgb200 {

constexpr int kTcMaxStages = 5;   // pipeline stages = generator groups; the launch picks as many as shared memory holds
constexpr int kTcMaxThreads = 32 * (4 * kTcMaxStages + 1);
constexpr int kTcStagedThreads = kTcMaxThreads + 32;   // + the warp that stages the generators' operands
constexpr int kOpRing = 16;       // ring entries (one per cell) the staging warp may run ahead of the generators
// ---------------------------------------------------------------------------------------------------------------
// Weight packing.  One block per cell: the T*T mid channels of the cell against all output channels of its degree,
// scaled by 1/max(eps, std), expanded to the real form, split into TF32 high and low parts and stored in the order
// the MMA descriptor expects (element (n', kk) at (n'/8)*(Kc/4)*32 + (kk/4)*32 + (n'%8)*4 + kk%4 floats), high part
// first.  One contiguous block per cell, so a stage's weights are a single bulk copy.
// ---------------------------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256)
tc_pack_kernel(PlanDev P, const int* __restrict__ npad, const int64_t* __restrict__ pack_off, const float2* __restrict__ W,
               const float* __restrict__ inv, float* __restrict__ pack) {
    constexpr int Kc = 2 * T * T;
    const int c = blockIdx.x;
    const CellInfo ci = P.cell_info[c];
    const int l = P.triples[P.cells[c].triple].l;
    const int N = npad[l];
    if (N == 0) return;
    const int to_n = P.tO[l], tff = P.tFF[l];
    float* hi = pack + pack_off[l] + (int64_t)(c - P.cell_begin[l]) * 2 * N * Kc;
    float* lo = hi + N * Kc;
    const float2* Wl = W + P.cumW[l];
    for (int e = threadIdx.x; e < N * Kc; e += blockDim.x) {
        const int np = e / Kc, kk = e - np * Kc;
        const int to = np >> 1, co = np & 1, idx = kk >> 1, cin = kk & 1;
        const int i = idx / T, j = idx - i * T;
        float v = 0.f;
        if (to < to_n && i < ci.v1 && j < ci.v2) {
            const int ch = i * ci.tau2 + j;
            const float2 w = __ldg(Wl + (int64_t)to * tff + ci.wch0 + ch);
            const float sc = __ldg(inv + ci.kch0 + ch);
            v = (co == 0 ? (cin == 0 ? w.x : -w.y) : (cin == 0 ? w.y : w.x)) * sc;
        }
        const float h = to_tf32(v);
        const int off = (np >> 3) * (Kc / 4) * 32 + (kk >> 2) * 32 + (np & 7) * 4 + (kk & 3);
        hi[off] = h;
        lo[off] = v - h;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The fused forward on the tensor cores.  grid = (row tiles, sample groups), 32 * (4 S + 1) threads.
// Dynamic shared memory: S x { A high [128 x Kc], A low [128 x Kc], B high+low [2 x n_max x Kc] } floats,
// then one CG band row per generator warp.
// ---------------------------------------------------------------------------------------------------------------

// KEPT: the generator warps load the tiles the statistics kernel of the same call kept (`ff`) instead of generating them
// (a separate instantiation, so that the generating kernel's register allocation is not touched by the extra path).
template <int T, bool KEPT>
__global__ void __launch_bounds__(kTcMaxThreads)
fused_fwd_tc_kernel(PlanDev P, const int* __restrict__ tiles, const int* __restrict__ npad, const int64_t* __restrict__ pack_off,
                    const float2* __restrict__ SF, const float* __restrict__ pack, float2* __restrict__ O,
                    float2* __restrict__ O_part, int64_t part_stride, int B, int n_max,
                    int max_n, int* __restrict__ status, int n_stages, int n_flush, uint32_t wait_limit, int idle_mma,
                    const float2* __restrict__ ff, int64_t ff_stride, const int64_t* __restrict__ ff_off) {
    constexpr int Kc = 2 * T * T;            // real K extent of one cell
    constexpr int NV = T * T;
    constexpr uint32_t kSbo = (Kc / 4) * 128;   // bytes between consecutive 8-row groups
    constexpr int kChunkCells = kChunkSteps / (3 * (Kc / 8));   // cells per chunk: three MMAs per K step of 8
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kTcMaxStages], empty_bar[kTcMaxStages], chunk_full[2], chunk_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;

    const int l = tiles[4 * blockIdx.x], m0 = tiles[4 * blockIdx.x + 1];
    const int part = tiles[4 * blockIdx.x + 2], parts = tiles[4 * blockIdx.x + 3];
    // group-major block order (all tiles of group 0, then group 1, ...): consecutive blocks on an SM read the same group's
    // slab, which the generators fetch through L1; tile-major order measured 30-60 % slower
    const int g = blockIdx.y;
    const int n = 2 * l + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this block's share of the degree's cells: k0 .. k0 + ncell - 1 (all of them unless the contraction is split)
    const int ncell_deg = P.cell_begin[l + 1] - P.cell_begin[l];
    const int k0 = (int)((int64_t)ncell_deg * part / parts);
    const int ncell = (int)((int64_t)ncell_deg * (part + 1) / parts) - k0;
    const int c_begin = P.cell_begin[l] + k0;
    const int N = npad[l];
    const int to_n = P.tO[l];
    const uint32_t tmem_cols = 4 * N <= 64 ? 64u : 4 * N <= 128 ? 128u : 4 * N <= 256 ? 256u : 512u;   // two regions of 2 N columns
    const size_t stage_floats = (size_t)2 * 128 * Kc + (size_t)2 * n_max * Kc;
    float* stages = reinterpret_cast<float*>(smem_raw);
    float* cbuf = stages + n_stages * stage_floats + (size_t)warp * max_n;
    const int gen_warps = 4 * n_stages;
    volatile int* failed = &failed_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 128);
            mbar_init(&empty_bar[s], 1);
        }
        for (int r = 0; r < 2; ++r) {
            mbar_init(&chunk_full[r], 1);
            mbar_init(&chunk_free[r], 4 * n_flush);   // one arrival per flush warp
        }
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < gen_warps) {
        // ---------------- generators ----------------
        const int s = warp >> 2, wq = warp & 3;
        const int mi = m0 + wq;
        const bool live_m = mi < n;
        const float2* slab = SF + (int64_t)g * P.nSF * 32 + lane;
        float* a_hi = stages + s * stage_floats;
        float* a_lo = a_hi + 128 * Kc;
        float* b_st = a_lo + 128 * Kc;
        const int r = wq * 32 + lane;
        float4* row_hi = reinterpret_cast<float4*>(a_hi) + (size_t)(r >> 3) * (Kc / 4) * 8 + (r & 7);
        float4* row_lo = reinterpret_cast<float4*>(a_lo) + (size_t)(r >> 3) * (Kc / 4) * 8 + (r & 7);
        const uint32_t b_bytes = (uint32_t)(2 * N * Kc * sizeof(float));
        bool ok = true;
        for (int k = s, u = 0; k < ncell && ok; k += n_stages, ++u) {
            if (u > 0) ok = mbar_wait_warp(&empty_bar[s], (uint32_t)((u - 1) & 1), failed, wait_limit);
            if (!ok) break;
            if (wq == 0 && lane == 0) {
                mbar_expect_tx(&full_bar[s], b_bytes);
                bulk_g2s(b_st, pack + pack_off[l] + (int64_t)(k0 + k) * 2 * N * Kc, b_bytes, &full_bar[s]);
            }
            float2 v[NV];
            if (KEPT && live_m) {
                // the statistics kernel of this call generated the tile already and kept it: [group][cell][m][entry][lane]
                const float2* src = ff + ((int64_t)g * ff_stride + ff_off[l] + ((int64_t)(k0 + k) * n + mi) * NV) * 32 + lane;
#pragma unroll
                for (int i = 0; i < NV; ++i) v[i] = src[i * 32];
            } else if (live_m) {
                const CellInfo ci = P.cell_info[c_begin + k];
                const int n2 = 2 * ci.l2 + 1;
                __syncwarp();
                for (int e = lane; e < n2; e += 32) cbuf[e] = __ldg(P.cg + ci.cgoff + mi * n2 + e);
                __syncwarp();
                gen_slab<T, false>(v, cbuf, slab + ci.o1 * 32, slab + ci.o2 * 32, mi - l, ci.l1, ci.l2);
            } else {
#pragma unroll
                for (int i = 0; i < NV; ++i) v[i] = make_float2(0.f, 0.f);
            }
#pragma unroll
            for (int q = 0; q < Kc / 4; ++q) {
                const float2 x0 = v[2 * q], x1 = v[2 * q + 1];
                float4 h, w;
                h.x = to_tf32(x0.x); h.y = to_tf32(x0.y); h.z = to_tf32(x1.x); h.w = to_tf32(x1.y);
                w.x = x0.x - h.x; w.y = x0.y - h.y; w.z = x1.x - h.z; w.w = x1.y - h.w;
                row_hi[q * 8] = h;
                row_lo[q * 8] = w;
            }
            fence_proxy_async();   // make the generic-proxy stores visible to the tensor core's async proxy
            mbar_arrive(&full_bar[s]);
        }
    } else if (warp == gen_warps) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && !idle_mma) {
            const uint32_t idesc = tc_idesc(128, N), idesc_wide = tc_idesc(128, 2 * N);
            bool ok = true;
            for (int k = 0; k < ncell && ok; ++k) {
                const int s = k % n_stages, u = k / n_stages;
                const int j = k / kChunkCells, r = j & 1;
                const bool first = k - j * kChunkCells == 0;
                // the flush warps have read this region's previous chunk (chunk j - 2)
                if (first && j >= 2) ok = mbar_wait(&chunk_free[r], (uint32_t)(((j >> 1) - 1) & 1), failed, wait_limit);
                if (!ok) break;
                ok = mbar_wait(&full_bar[s], (uint32_t)(u & 1), failed, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(r * 2 * N);
                const uint32_t a_hi = smem_u32(stages + s * stage_floats);
                const uint32_t a_lo = a_hi + 128 * Kc * 4;
                const uint32_t b_hi = a_lo + 128 * Kc * 4;   // high part; the low part follows as rows N .. 2 N - 1 of the same K-major matrix
                const uint64_t dah0 = smem_desc(a_hi, 128, kSbo), dal0 = smem_desc(a_lo, 128, kSbo);
                const uint64_t dbh0 = smem_desc(b_hi, 128, kSbo);
#pragma unroll
                for (int ks = 0; ks < Kc / 8; ++ks) {
                    const uint64_t dah = desc_advance(dah0, ks * 256), dal = desc_advance(dal0, ks * 256);
                    const uint64_t dbh = desc_advance(dbh0, ks * 256);
                    tc_mma_tf32(d, dah, dbh, idesc_wide, (!first || ks > 0) ? 1u : 0u);   // Ah x [Bh | Bl] -> columns 0 .. 2 N
                    tc_mma_tf32(d, dal, dbh, idesc, 1u);                                   // Al x Bh       -> columns 0 .. N
                }
                tc_commit(&empty_bar[s]);   // arrives when the MMAs above have finished reading the stage
                if (k - j * kChunkCells == kChunkCells - 1 || k == ncell - 1) tc_commit(&chunk_full[r]);   // chunk j is summed
            }
        }
    } else {
        // ---------------- flush warps: running sums in registers, then the output ----------------
        const int fw = warp - gen_warps - 1;          // 0 .. 4 n_flush - 1
        const int fg = fw >> 2;                       // flush group: columns [64 fg, 64 fg + 64) of the accumulator
        const int wq = warp & 3;                      // the TMEM lane quarter this warp may read = its m inside the row tile
        const int mi = m0 + wq;
        const bool live_m = mi < n;
        const int col_base = 64 * fg;
        const int n_chunks = (ncell + kChunkCells - 1) / kChunkCells;
        float run[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) run[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_chunks && ok; ++j) {
            const int r = j & 1;
            ok = mbar_wait_warp(&chunk_full[r], (uint32_t)((j >> 1) & 1), failed, wait_limit);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const int col0 = col_base + 16 * c4;
                if (col0 < N) {   // warp-uniform
                    uint32_t rr[16], rl[16];   // the chunk's Ah Bh + Al Bh and its Ah Bl
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * 2 * N + col0), rr);
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * 2 * N + N + col0), rl);
#pragma unroll
                    for (int i = 0; i < 16; ++i) run[16 * c4 + i] += __uint_as_float(rr[i]) + __uint_as_float(rl[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&chunk_free[r]);   // the region may be overwritten by chunk j + 2
        }
        const int b = g * 32 + lane;
        if (live_m && b < B) {
            float2* out = (parts > 1 ? O_part + (int64_t)part * part_stride : O) + (int64_t)b * P.n_O + P.cumO[l] + mi;
            const float nanv = __uint_as_float(kNaNBits);   // a block that gave up marks the outputs it owns
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int to = ((col_base + 16 * c4) >> 1) + i;
                    if (to < to_n) out[(int64_t)to * n] = ok ? make_float2(run[16 * c4 + 2 * i], run[16 * c4 + 2 * i + 1]) : make_float2(nanv, nanv);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// The same forward with everything a cell needs staged in shared memory ahead of time.
//
// Measured on the kernel above (lmax 10, 16 channels): with generation and MMAs both switched off, the skeleton alone -
// per cell: wait for the stage, start the bulk copy of the cell's weights into it, store the A tile, wait for the copy,
// issue, wait for completion - took half of the kernel's time, because the stage's chain "free -> weights copy -> MMA ->
// free" is serial and the copy's latency (about 1.5 us from L2) sits in it once per cell; the generator's operand loads
// from L2 (the slab of a sample group is far larger than L1) came second; the MMAs themselves were 10 %.
// Here a staging warp runs up to kOpRing cells ahead of the generators and puts, per cell, into one entry of a byte ring:
//   the four CG band rows of the block's m (one cp.async.bulk from a copy of the table whose rows are padded to 16 bytes),
//   the rows of the two operand tiles those m can touch (two cp.async.bulk from the slab: they are contiguous there),
//   the cell's packed weights (one cp.async.bulk),
// with one mbarrier per entry counting the staging warp's arrival and the copies' bytes.  The generators read their
// operands from shared memory, compute the tile in registers *before* they wait for their A stage to be free, and the
// MMA warp takes the B operand straight from the ring entry; the entry goes back to the staging warp when the four
// generator warps and the cell's MMAs (tcgen05.commit) are done with it.  A stage holds only the A tile.
// ---------------------------------------------------------------------------------------------------------------
struct OpEntry {
    int band;         // ring offset (floats) of the four band rows, row stride (2 l2 + 1) rounded up to a multiple of 4
    int s1, s2;       // ring offset (float2) of the t1 tile's / t2 tile's virtual row 0 (the fragment's m = -l)
    int wgt;          // ring offset (floats) of the packed weights: high part, then low part
    short l1, l2;
};

template <int T>
__global__ void __launch_bounds__(kTcStagedThreads)
fused_fwd_tc_staged_kernel(PlanDev P, const int* __restrict__ tiles, const int* __restrict__ npad,
                           const int64_t* __restrict__ pack_off, const float* __restrict__ cg_pad, const int* __restrict__ cell_cgpad,
                           const float2* __restrict__ SF, const float* __restrict__ pack,
                           float2* __restrict__ O, int B, int* __restrict__ status, int n_stages, int n_abuf, int n_flush,
                           int ring_bytes, int stage_rows, uint32_t wait_limit, int idle_mma) {
    constexpr int Kc = 2 * T * T;            // real K extent of one cell
    constexpr int NV = T * T;
    constexpr uint32_t kSbo = (Kc / 4) * 128;   // bytes between consecutive 8-row groups
    constexpr int kChunkCells = kChunkSteps / (3 * (Kc / 8));
    constexpr int kRow = T * 32;             // float2 per operand row (T channels x 32 samples)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kTcMaxStages], empty_bar[kTcMaxStages], chunk_full[2], chunk_free[2];
    __shared__ __align__(8) uint64_t op_full[kOpRing], op_empty[kOpRing];
    __shared__ OpEntry op_tab[kOpRing];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;

    const int l = tiles[4 * blockIdx.x], m0 = tiles[4 * blockIdx.x + 1];   // level 0 of the tile lists: whole contractions
    const int g = blockIdx.y;
    const int n = 2 * l + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c_begin = P.cell_begin[l], ncell = P.cell_begin[l + 1] - c_begin;
    const int N = npad[l];
    const int to_n = P.tO[l];
    const uint32_t tmem_cols = 4 * N <= 64 ? 64u : 4 * N <= 128 ? 128u : 4 * N <= 256 ? 256u : 512u;   // two regions of 2 N columns
    constexpr size_t stage_floats = (size_t)2 * 128 * Kc;   // A tile, high and low part
    float* stages = reinterpret_cast<float*>(smem_raw);
    unsigned char* ring = smem_raw + (size_t)n_abuf * stage_floats * sizeof(float);
    float* ringf = reinterpret_cast<float*>(ring);
    float2* ring2 = reinterpret_cast<float2*>(ring);
    const int gen_warps = 4 * n_stages;
    volatile int* failed = &failed_flag;

    if (threadIdx.x == 0) {
        for (int a = 0; a < n_abuf; ++a) {
            mbar_init(&full_bar[a], 4);      // one arrival per generator warp
            mbar_init(&empty_bar[a], 1);
        }
        for (int r = 0; r < 2; ++r) {
            mbar_init(&chunk_full[r], 1);
            mbar_init(&chunk_free[r], 4 * n_flush);
        }
        for (int e = 0; e < kOpRing; ++e) {
            mbar_init(&op_full[e], 1);     // the staging warp's arrival + the bytes of its copies
            mbar_init(&op_empty[e], 5);    // four generator warps + the completion of the cell's MMAs
        }
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < gen_warps) {
        // ---------------- generators ----------------
        const int s = warp >> 2, wq = warp & 3;
        const int mi = m0 + wq;
        const bool live_m = mi < n;
        const float2* slab = SF + (int64_t)g * P.nSF * 32 + lane;   // this lane's view of the group's slab (operands not staged)
        const int r = wq * 32 + lane;
        const size_t row_off = (size_t)(r >> 3) * (Kc / 4) * 8 + (r & 7);   // this lane's row inside an A tile, in float4
        bool ok = true;
        // group s generates the cells s, s + S, ...; cell k goes to A buffer k % n_abuf (more buffers than groups: a group
        // stores its next tile while the MMAs of its previous one are still in flight)
        for (int k = s; k < ncell && ok; k += n_stages) {
            const int e = k % kOpRing;
            const int ab = k % n_abuf, ua = k / n_abuf;
            float4* row_hi = reinterpret_cast<float4*>(stages + ab * stage_floats) + row_off;
            float4* row_lo = row_hi + 128 * Kc / 4;
            ok = mbar_wait_warp(&op_full[e], (uint32_t)((k / kOpRing) & 1), failed, wait_limit);   // the cell's entry is staged
            if (!ok) break;
            float2 v[NV];
            if (live_m) {
                const OpEntry oe = op_tab[e];
                const float* crow = ringf + oe.band + wq * ((2 * oe.l2 + 4) & ~3);
                if (stage_rows) gen_slab<T, false>(v, crow, ring2 + oe.s1 + lane, ring2 + oe.s2 + lane, mi - l, oe.l1, oe.l2);
                else gen_slab<T, false, true>(v, crow, slab + (int64_t)oe.s1 * 32, slab + (int64_t)oe.s2 * 32, mi - l, oe.l1, oe.l2);
            } else {
#pragma unroll
                for (int i = 0; i < NV; ++i) v[i] = make_float2(0.f, 0.f);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&op_empty[e]);   // this warp is done reading the entry
            if (ua > 0) ok = mbar_wait_warp(&empty_bar[ab], (uint32_t)((ua - 1) & 1), failed, wait_limit);   // the buffer's previous MMAs are done
            if (!ok) break;
#pragma unroll
            for (int q = 0; q < Kc / 4; ++q) {
                const float2 x0 = v[2 * q], x1 = v[2 * q + 1];
                float4 h, w;
                h.x = to_tf32(x0.x); h.y = to_tf32(x0.y); h.z = to_tf32(x1.x); h.w = to_tf32(x1.y);
                w.x = x0.x - h.x; w.y = x0.y - h.y; w.z = x1.x - h.z; w.w = x1.y - h.w;
                row_hi[q * 8] = h;
                row_lo[q * 8] = w;
            }
            fence_proxy_async();   // make the generic-proxy stores visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[ab]);
        }
    } else if (warp == gen_warps) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && !idle_mma) {
            const uint32_t idesc = tc_idesc(128, N), idesc_wide = tc_idesc(128, 2 * N);
            bool ok = true;
            for (int k = 0; k < ncell && ok; ++k) {
                const int s = k % n_abuf, u = k / n_abuf;   // A buffer of the cell and its use count
                const int e = k % kOpRing;
                const int j = k / kChunkCells, r = j & 1;
                const bool first = k - j * kChunkCells == 0;
                if (first && j >= 2) ok = mbar_wait(&chunk_free[r], (uint32_t)(((j >> 1) - 1) & 1), failed, wait_limit);
                if (!ok) break;
                ok = mbar_wait(&op_full[e], (uint32_t)((k / kOpRing) & 1), failed, wait_limit);   // the weights have landed
                if (!ok) break;
                const uint32_t wgt = smem_u32(ringf + op_tab[e].wgt);
                ok = mbar_wait(&full_bar[s], (uint32_t)(u & 1), failed, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(r * 2 * N);
                const uint32_t a_hi = smem_u32(stages + s * stage_floats);
                const uint32_t a_lo = a_hi + 128 * Kc * 4;
                const uint32_t b_hi = wgt;   // high part; the low part follows as rows N .. 2 N - 1 of the same K-major matrix
                const uint64_t dah0 = smem_desc(a_hi, 128, kSbo), dal0 = smem_desc(a_lo, 128, kSbo);
                const uint64_t dbh0 = smem_desc(b_hi, 128, kSbo);
#pragma unroll
                for (int ks = 0; ks < Kc / 8; ++ks) {
                    const uint64_t dah = desc_advance(dah0, ks * 256), dal = desc_advance(dal0, ks * 256);
                    const uint64_t dbh = desc_advance(dbh0, ks * 256);
                    tc_mma_tf32(d, dah, dbh, idesc_wide, (!first || ks > 0) ? 1u : 0u);   // Ah x [Bh | Bl] -> columns 0 .. 2 N
                    tc_mma_tf32(d, dal, dbh, idesc, 1u);                                   // Al x Bh       -> columns 0 .. N
                }
                tc_commit(&empty_bar[s]);    // the MMAs above have finished reading the A stage ...
                tc_commit(&op_empty[e]);     // ... and the entry's weights
                if (k - j * kChunkCells == kChunkCells - 1 || k == ncell - 1) tc_commit(&chunk_full[r]);
            }
        }
    } else if (warp == gen_warps + 1) {
        // ---------------- staging warp ----------------
        // All lanes run the ring bookkeeping alike (the waits are warp-wide); lane 0 issues the copies.  The cell records
        // are fetched 32 at a time, one per lane, a batch ahead of their use, and handed out by shuffles.
        const int mt_lo = m0 - l, mt_hi = min(m0 + 3, n - 1) - l;   // the block's m values
        const int mrows = mt_hi - mt_lo + 1;
        const float2* slab0 = SF + (int64_t)g * P.nSF * 32;
        const int ring_f2 = ring_bytes / 8;
        const uint32_t wgt_bytes = (uint32_t)(2 * N * Kc * sizeof(float));
        int start[kOpRing];     // ring offset (float2) where each live entry begins
        int head = 0, tail = 0; // the live entries occupy [tail, head) of the ring, circularly
        int kt = 0;             // oldest cell whose entry has not been handed back
        int last = -1;          // newest cell staged
        bool ok = true;
        // this lane's cell of the current and of the next batch: (o1, o2, l1 | l2 << 16, padded band offset)
        int4 cur = make_int4(0, 0, 0, 0), nxt = make_int4(0, 0, 0, 0);
        auto fetch = [&](int k0) -> int4 {
            const int c = k0 + lane;
            if (c >= ncell) return make_int4(0, 0, 0, 0);
            const CellInfo x = P.cell_info[c_begin + c];
            return make_int4(x.o1, x.o2, (int)x.l1 | ((int)x.l2 << 16), cell_cgpad[c_begin + c]);
        };
        nxt = fetch(0);
        for (int k = 0; k < ncell && ok; ++k) {
            if ((k & 31) == 0) {
                cur = nxt;
                nxt = fetch(k + 32);
            }
            const int src = k & 31;
            const int o1 = __shfl_sync(0xffffffffu, cur.x, src), o2 = __shfl_sync(0xffffffffu, cur.y, src);
            const int ll = __shfl_sync(0xffffffffu, cur.z, src), cgp = __shfl_sync(0xffffffffu, cur.w, src);
            const int l1 = ll & 0xffff, l2 = ll >> 16, n2p = (2 * l2 + 4) & ~3;
            // rows (m index + l of the fragment) the block's m values touch: m1 = m - m2, m2 over the band
            const int r1_lo = max(-l1, mt_lo - l2) + l1, r1_hi = min(l1, mt_hi + l2) + l1;
            const int r2_lo = max(-l2, mt_lo - l1) + l2, r2_hi = min(l2, mt_hi + l1) + l2;
            const int n1r = stage_rows ? (r1_hi - r1_lo + 1) * kRow : 0, n2r = stage_rows ? (r2_hi - r2_lo + 1) * kRow : 0;   // float2 per tile
            const int band_f2 = ((4 * n2p + 31) & ~31) / 2;                                    // 128-byte granules
            const int need = band_f2 + n1r + n2r + (int)(wgt_bytes / 8);
            int at = -1;
            while (ok) {
                if (k - kt < kOpRing) {
                    if (kt == k) { head = tail = 0; at = 0; }                          // nothing live: start over
                    else if (head >= tail) {
                        if (head + need <= ring_f2) at = head;
                        else if (need < tail) at = 0;                                   // wrap: the gap at the end stays unused
                    } else if (head + need < tail) at = head;
                    if (at >= 0) break;
                }
                // entries come back in cell order as far as this warp is concerned: wait for the oldest live one
                ok = mbar_wait_warp(&op_empty[kt % kOpRing], (uint32_t)((kt / kOpRing) & 1), failed, wait_limit);
                ++kt;
                tail = kt < k ? start[kt % kOpRing] : head;
            }
            if (!ok) break;
            const int e = k % kOpRing;
            start[e] = at;
            head = at + need;
            if (kt == k) tail = at;
            if (lane == 0) {
                OpEntry oe;
                oe.band = 2 * at;
                oe.s1 = stage_rows ? at + band_f2 - r1_lo * kRow : o1;   // ring offset of the staged rows, or the tile's slab offset
                oe.s2 = stage_rows ? at + band_f2 + n1r - r2_lo * kRow : o2;
                oe.wgt = 2 * (at + band_f2 + n1r + n2r);
                oe.l1 = (short)l1;
                oe.l2 = (short)l2;
                op_tab[e] = oe;
                const uint32_t band_bytes = (uint32_t)(mrows * n2p) * 4u;
                // release: the table entry becomes visible to the waiters
                mbar_arrive_expect_tx(&op_full[e], band_bytes + (uint32_t)(n1r + n2r) * 8u + wgt_bytes);
                bulk_g2s(ringf + oe.band, cg_pad + cgp + m0 * n2p, band_bytes, &op_full[e]);
                if (stage_rows) {
                    bulk_g2s(ring2 + at + band_f2, slab0 + (int64_t)(o1 + r1_lo * T) * 32, (uint32_t)n1r * 8u, &op_full[e]);
                    bulk_g2s(ring2 + at + band_f2 + n1r, slab0 + (int64_t)(o2 + r2_lo * T) * 32, (uint32_t)n2r * 8u, &op_full[e]);
                }
                bulk_g2s(ringf + oe.wgt, pack + pack_off[l] + (int64_t)k * 2 * N * Kc, wgt_bytes, &op_full[e]);
            }
            last = k;
        }
        // a block that gave up may leave before the newest entries were consumed: let their copies land first
        if (lane == 0 && (!ok || *failed))
            for (int k = max(0, last - kOpRing + 1); k <= last; ++k) mbar_drain(&op_full[k % kOpRing], (uint32_t)((k / kOpRing) & 1), wait_limit);
    } else {
        // ---------------- flush warps: running sums in registers, then the output ----------------
        const int fw = warp - gen_warps - 2;          // 0 .. 4 n_flush - 1
        const int fg = fw >> 2;                       // flush group: columns [64 fg, 64 fg + 64) of the accumulator
        const int wq = warp & 3;                      // the TMEM lane quarter this warp may read = its m inside the row tile
        const int mi = m0 + wq;
        const bool live_m = mi < n;
        const int col_base = 64 * fg;
        const int n_chunks = (ncell + kChunkCells - 1) / kChunkCells;
        float run[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) run[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_chunks && ok; ++j) {
            const int r = j & 1;
            ok = mbar_wait_warp(&chunk_full[r], (uint32_t)((j >> 1) & 1), failed, wait_limit);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const int col0 = col_base + 16 * c4;
                if (col0 < N) {   // warp-uniform
                    uint32_t rr[16], rl[16];   // the chunk's Ah Bh + Al Bh and its Ah Bl
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * 2 * N + col0), rr);
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * 2 * N + N + col0), rl);
#pragma unroll
                    for (int i = 0; i < 16; ++i) run[16 * c4 + i] += __uint_as_float(rr[i]) + __uint_as_float(rl[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&chunk_free[r]);   // the region may be overwritten by chunk j + 2
        }
        const int b = g * 32 + lane;
        if (live_m && b < B) {
            float2* out = O + (int64_t)b * P.n_O + P.cumO[l] + mi;
            const float nanv = __uint_as_float(kNaNBits);   // a block that gave up marks the outputs it owns
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int to = ((col_base + 16 * c4) >> 1) + i;
                    if (to < to_n) out[(int64_t)to * n] = ok ? make_float2(run[16 * c4 + 2 * i], run[16 * c4 + 2 * i + 1]) : make_float2(nanv, nanv);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// The weight gradient on the tensor cores.
//
//   gW_l[to, k] = 1/std_k * sum_{b, m} conj(FF_l[b, k, m]) * gO_l[b, to, m]
//
// as a real GEMM that contracts over (m, b):  D[(k, re|im), (to, re|im)] = sum A'[(k, .), (m, b)] * B'[(to, .), (m, b)],
// from which gW.re = D[kr, tor] + D[ki, toi] and gW.im = D[kr, toi] - D[ki, tor].  Block = four cells (tile edge 4) or two
// cells (tile edge 5) of one degree = up to 128 rows of D = the 128 lanes of tensor memory, against all output channels;
// it walks every (sample group of its slice, m), 32 samples = one K chunk = four K steps of the MMA.  Generator group s
// (four warps, see GwTcShape) fills pipeline stage s for the chunks s, s + S, ...: the cell's FF values of its lane's
// sample, split into TF32 high / low parts, go to shared memory as the M x K operand (K-major: a lane owns one K
// column), and the four warps share the chunk's gO values as the N x K operand.  The K stride between core matrices is
// 144 bytes instead of 128, so that the eight lane quads of a warp, which write eight different core matrices of the
// same row, fall into different banks.  MMA warp, barriers, bounded waits and 3xTF32 as in the forward kernel; the
// accumulation order is fixed, so the result is bit-identical from run to run.
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t kGwLbo = 144;           // bytes between K-adjacent core matrices (8 rows x 16 bytes, then 16 bytes of padding)
constexpr uint32_t kGwSbo = 8 * kGwLbo;    // bytes between 8-row groups: a K chunk of 32 samples = 8 core matrices

// Shape of a weight-gradient block by tile edge.  Tile edge 4: four cells of 32 real rows, one generator warp per cell.
// Tile edge 5: two cells of 50 real rows (100 of the 128 accumulator rows used), two generator warps per cell, each
// with half the tile's rows (3 + 2), which also halves the registers of the generator.
template <int T>
struct GwTcShape {
    static constexpr int NV = T * T;
    static constexpr int MR = 2 * NV;            // real rows of D per cell
    static constexpr int kCells = 128 / MR;      // cells per block
    static constexpr int kSplit = 4 / kCells;    // generator warps per cell
    static_assert(kCells * kSplit == 4 && kCells * MR <= 128, "a generator group is four warps");
};

// one generator warp's values of a chunk: rows [I0, I0 + IN) of cell `c`'s tile -> TF32 high / low parts in the A' stage
// (`tile`: the row's kept values, [tile entry][32 lanes] with the lane already added, or null to generate them)
template <int T, int I0, int IN>
__device__ __forceinline__ void gw_tc_generate(const CellInfo& ci, const float2* __restrict__ slab, const float* __restrict__ cbuf,
                                               int mi, int l, int c, unsigned char* __restrict__ a_hi, uint32_t a_bytes,
                                               const float2* __restrict__ tile) {
    constexpr int MR = 2 * T * T;
    float2 v[IN * T];
    if (tile != nullptr) {
#pragma unroll
        for (int e = 0; e < IN * T; ++e) v[e] = tile[(I0 * T + e) * 32];
    } else if constexpr (IN == T) {
        gen_slab<T, false, true>(v, cbuf, slab + ci.o1 * 32, slab + ci.o2 * 32, mi - l, ci.l1, ci.l2);
    } else {
        gen_slab_rows<T, I0, IN>(v, cbuf, slab + ci.o1 * 32, slab + ci.o2 * 32, mi - l, ci.l1, ci.l2);
    }
    const int rbase = c * MR + 2 * I0 * T;   // even: a value's (re, im) rows share an 8-row group
#pragma unroll
    for (int e = 0; e < IN * T; ++e) {
        const int r = rbase + 2 * e;
        unsigned char* ph = a_hi + (uint32_t)(r >> 3) * kGwSbo + (uint32_t)(r & 7) * 16;
        const float hx = to_tf32(v[e].x), hy = to_tf32(v[e].y);
        *reinterpret_cast<float*>(ph) = hx;
        *reinterpret_cast<float*>(ph + 16) = hy;
        *reinterpret_cast<float*>(ph + a_bytes) = v[e].x - hx;
        *reinterpret_cast<float*>(ph + a_bytes + 16) = v[e].y - hy;
    }
}

// grid = (blocks of cells, slices of the sample groups); slice s handles the groups s, s + slices, ... and, with more
// than one slice, writes its partial sums to gW + s * slice_stride for gw_reduce_kernel
template <int T, bool KEPT>
__global__ void __launch_bounds__(kTcMaxThreads)
fused_gw_tc_kernel(PlanDev P, const int* __restrict__ tiles, const int* __restrict__ npad, const float2* __restrict__ SF,
                   const float2* __restrict__ SG, const float* __restrict__ inv, float2* __restrict__ gW, int G, int n_max,
                   int max_n, int* __restrict__ status, int n_stages, int n_flush, int64_t slice_stride, uint32_t wait_limit,
                   int idle_mma, const float2* __restrict__ ff, int64_t ff_stride, const int64_t* __restrict__ ff_off) {
    using S = GwTcShape<T>;
    constexpr int MR = S::MR;
    constexpr int kFlushChunks = kChunkSteps / 12;   // K chunks (32 samples = 4 K steps x 3 MMAs) summed in tensor memory before a flush
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kTcMaxStages], empty_bar[kTcMaxStages], chunk_full[2], chunk_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;

    const int l = tiles[2 * blockIdx.x], cell0 = tiles[2 * blockIdx.x + 1];
    const int slice = blockIdx.y, slices = gridDim.y;
    const int n = 2 * l + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c_begin = P.cell_begin[l], ncell = P.cell_begin[l + 1] - c_begin;
    const int N = npad[l];
    const int to_n = P.tO[l], tff = P.tFF[l];
    const uint32_t tmem_cols = 2 * N <= 32 ? 32u : 2 * N <= 64 ? 64u : 2 * N <= 128 ? 128u : 256u;   // two regions of N columns
    const uint32_t a_bytes = 16 * kGwSbo, b_bytes = (uint32_t)(n_max / 8) * kGwSbo;
    const uint32_t stage_bytes = 2 * a_bytes + 2 * b_bytes;
    float* cbuf = reinterpret_cast<float*>(smem_raw + (size_t)n_stages * stage_bytes) + (size_t)warp * max_n;
    const int gen_warps = 4 * n_stages;
    const int n_groups = slice < G ? (G - slice + slices - 1) / slices : 0;   // sample groups of this slice
    const int n_chunks = n * n_groups;
    volatile int* failed = &failed_flag;
    float2* __restrict__ out_base = gW + (int64_t)slice * slice_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 128);
            mbar_init(&empty_bar[s], 1);
        }
        for (int r = 0; r < 2; ++r) {
            mbar_init(&chunk_full[r], 1);
            mbar_init(&chunk_free[r], 4 * n_flush);   // one arrival per flush warp
        }
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < gen_warps) {
        // ---------------- generators ----------------
        const int s = warp >> 2, wq = warp & 3;
        const int c = wq / S::kSplit, half = wq % S::kSplit;   // cell of the block, part of its rows
        const int cell = cell0 + c;
        const bool live = cell < ncell;
        CellInfo ci{};
        if (live) ci = P.cell_info[c_begin + cell];
        const int n2 = 2 * ci.l2 + 1;
        unsigned char* st_base = smem_raw + (size_t)s * stage_bytes;
        // this lane's K column inside a chunk: core matrix lane/4 along K, word lane%4 inside its 16-byte row
        const uint32_t col_off = (uint32_t)(lane >> 2) * kGwLbo + (uint32_t)(lane & 3) * 4;
        unsigned char* a_hi = st_base + col_off;
        unsigned char* b_hi = st_base + 2 * a_bytes + col_off;
        unsigned char* b_lo = b_hi + b_bytes;
        const int to_per = (to_n + 3) >> 2, to_lo = wq * to_per, to_hi = min(to_n, to_lo + to_per);
        bool ok = true;
        for (int q = s, u = 0; q < n_chunks && ok; q += n_stages, ++u) {
            if (u > 0) ok = mbar_wait_warp(&empty_bar[s], (uint32_t)((u - 1) & 1), failed, wait_limit);
            if (!ok) break;
            const int gi = q / n, mi = q - gi * n;
            const int g = slice + gi * slices;
            if (live) {
                const float2* slab = SF + (int64_t)g * P.nSF * 32 + lane;
                // the tiles the forward kept (same generator, same bits), or the band row to generate them again
                const float2* tile = !KEPT ? nullptr
                                           : ff + ((int64_t)g * ff_stride + ff_off[l] + ((int64_t)cell * n + mi) * S::NV) * 32 + lane;
                if (tile == nullptr) {
                    __syncwarp();
                    for (int e = lane; e < n2; e += 32) cbuf[e] = __ldg(P.cg + ci.cgoff + mi * n2 + e);
                    __syncwarp();
                }
                if constexpr (S::kSplit == 1) {
                    gw_tc_generate<T, 0, T>(ci, slab, cbuf, mi, l, c, a_hi, a_bytes, tile);
                } else {
                    constexpr int AH = (T + 1) / 2;
                    if (half == 0) gw_tc_generate<T, 0, AH>(ci, slab, cbuf, mi, l, c, a_hi, a_bytes, tile);
                    else gw_tc_generate<T, AH, T - AH>(ci, slab, cbuf, mi, l, c, a_hi, a_bytes, tile);
                }
            }
            const float2* go = SG + ((int64_t)g * P.nSO + P.cumSO[l]) * 32 + lane;
            for (int to = to_lo; to < to_hi; ++to) {
                const float2 gv = go[(((to / T) * n + mi) * T + to % T) * 32];
                const float hr = to_tf32(gv.x), hi_ = to_tf32(gv.y);
                const int r0 = 2 * to;   // rows (to, re) and (to, im): same 8-row group, adjacent 16-byte rows
                const uint32_t off = (uint32_t)(r0 >> 3) * kGwSbo + (uint32_t)(r0 & 7) * 16;
                *reinterpret_cast<float*>(b_hi + off) = hr;
                *reinterpret_cast<float*>(b_hi + off + 16) = hi_;
                *reinterpret_cast<float*>(b_lo + off) = gv.x - hr;
                *reinterpret_cast<float*>(b_lo + off + 16) = gv.y - hi_;
            }
            fence_proxy_async();   // make the generic-proxy stores visible to the tensor core's async proxy
            mbar_arrive(&full_bar[s]);
        }
    } else if (warp == gen_warps) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && !idle_mma) {
            const uint32_t idesc = tc_idesc(128, N);
            bool ok = true;
            for (int q = 0; q < n_chunks && ok; ++q) {
                const int s = q % n_stages, u = q / n_stages;
                const int j = q / kFlushChunks, r = j & 1;
                const bool first = q - j * kFlushChunks == 0;
                // the flush warps have read this region's previous contents (flush chunk j - 2)
                if (first && j >= 2) ok = mbar_wait(&chunk_free[r], (uint32_t)(((j >> 1) - 1) & 1), failed, wait_limit);
                if (!ok) break;
                ok = mbar_wait(&full_bar[s], (uint32_t)(u & 1), failed, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(r * N);
                const uint32_t a_hi = smem_u32(smem_raw + (size_t)s * stage_bytes);
                const uint32_t a_lo = a_hi + a_bytes;
                const uint32_t b_hi = a_lo + a_bytes;
                const uint32_t b_lo = b_hi + b_bytes;
                const uint64_t dah0 = smem_desc(a_hi, kGwLbo, kGwSbo), dal0 = smem_desc(a_lo, kGwLbo, kGwSbo);
                const uint64_t dbh0 = smem_desc(b_hi, kGwLbo, kGwSbo), dbl0 = smem_desc(b_lo, kGwLbo, kGwSbo);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {   // 32 samples = 4 K steps of 8 = 2 core matrices each
                    const uint32_t koff = ks * 2 * kGwLbo;
                    const uint64_t dah = desc_advance(dah0, koff), dal = desc_advance(dal0, koff);
                    const uint64_t dbh = desc_advance(dbh0, koff), dbl = desc_advance(dbl0, koff);
                    tc_mma_tf32(d, dah, dbh, idesc, (!first || ks > 0) ? 1u : 0u);
                    tc_mma_tf32(d, dal, dbh, idesc, 1u);
                    tc_mma_tf32(d, dah, dbl, idesc, 1u);
                }
                tc_commit(&empty_bar[s]);   // arrives when the MMAs above have finished reading the stage
                if (q - j * kFlushChunks == kFlushChunks - 1 || q == n_chunks - 1) tc_commit(&chunk_full[r]);
            }
        }
    } else {
        // ---------------- flush warps: running sums of the accumulator in registers, then gW ----------------
        // (the tensor core adds into its accumulator with truncation: long contractions are summed in pieces, see the
        // forward kernel).  Warp w reads accumulator rows 32 (w % 4) .. + 31; flush group fg owns columns [64 fg, 64 fg + 64).
        const int fw = warp - gen_warps - 1;
        const int fg = fw >> 2;
        const int wq = warp & 3;
        const int col_base = 64 * fg;
        const int n_flushes = (n_chunks + kFlushChunks - 1) / kFlushChunks;
        float run[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) run[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_flushes && ok; ++j) {
            const int r = j & 1;
            ok = mbar_wait_warp(&chunk_full[r], (uint32_t)((j >> 1) & 1), failed, wait_limit);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const int col0 = col_base + 16 * c4;
                if (col0 < N) {   // warp-uniform
                    uint32_t rr[16];
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * N + col0), rr);
#pragma unroll
                    for (int i = 0; i < 16; ++i) run[16 * c4 + i] += __uint_as_float(rr[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&chunk_free[r]);
        }
        const int row = wq * 32 + lane;
        const int ec = row / MR, kk = row - ec * MR;   // cell of the block and real row inside it
        const int idx = kk >> 1, i = idx / T, jj = idx - i * T;
        CellInfo ei{};
        const bool e_live = ec < S::kCells && cell0 + ec < ncell;
        if (e_live) ei = P.cell_info[c_begin + cell0 + ec];
        const bool writer = e_live && (kk & 1) == 0 && i < ei.v1 && jj < ei.v2;
        const int ch = i * ei.tau2 + jj;
        const float sc = writer ? inv[ei.kch0 + ch] : 0.f;
        float2* out = out_base + P.cumW[l] + ei.wch0 + ch;
        const float nanv = __uint_as_float(kNaNBits);   // a block that gave up marks the outputs it owns
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                const float mr = ok ? run[16 * c4 + 2 * cc] : nanv, mim = ok ? run[16 * c4 + 2 * cc + 1] : nanv;
                const float orr = __shfl_xor_sync(0xffffffffu, mr, 1), oim = __shfl_xor_sync(0xffffffffu, mim, 1);
                const int to = ((col_base + 16 * c4) >> 1) + cc;
                // even lane = row (k, re), its neighbour = row (k, im)
                if (writer && to < to_n) out[(int64_t)to * tff] = make_float2((mr + oim) * sc, (mim - orr) * sc);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// The input gradient with its first phase on the tensor cores.
//
// Same block structure, entry walk, staging and phase 2 as fused_gf_kernel (fused.cu); what changes is phase 1, the
// gFF tile  H[(m, b), k] = sum_to conj(W[to, k])/std_k * gO[b, to, m]:  it is the real GEMM
//   D[(m, b), (k, re|im)] = sum_{(to, re|im)} G[(m, b), (to, re|im)] * Bw[(k, re|im), (to, re|im)]
// with 128 rows = four m x 32 samples per MMA tile and the 2T^2 = 32 real columns of one cell.  Per (row tile, chunk
// of 16 output channels) the 16 warps write the gO values of their lanes' samples, split into TF32 high / low parts,
// into one of two shared-memory A buffers (a lane owns a row: 16-byte stores, no conflicts); after a block barrier one
// thread issues the 4 x 3 tcgen05.mma (3xTF32) of the chunk into the tile's 32 tensor-memory columns and commits them
// to the buffer's "empty" barrier, so the next chunk is staged while this one is multiplied.  The weights of the entry
// (real form of conj(W)/std, high / low parts) are the B operand, written once per entry.  When the entry's last MMA has
// completed, the warps move H from tensor memory to the shared-memory transit buffer (warp w can read the rows
// with m % 4 == w % 4) in chunks of Mc m's and run phase 2 on every chunk exactly as the CUDA-core kernel does.
// All waits are bounded; a wait that runs out sets the plan's status word and the block finishes without hanging.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool mbar_wait_checked(uint64_t* bar, uint32_t parity, volatile int* failed, uint32_t limit) {
    if (__any_sync(0xffffffffu, *failed)) return false;   // warp-uniform
    return mbar_wait_warp(bar, parity, failed, limit);
}

template <int T>
__global__ void __launch_bounds__(kGfWarps * 32)
fused_gf_tc_kernel(PlanDev P, const GfInfo* __restrict__ entries, const int* __restrict__ entry_begin,
                   const int* __restrict__ blocks, const unsigned char* __restrict__ owner_tab, const float2* __restrict__ SF,
                   const float2* __restrict__ SG, const float2* __restrict__ W, const float* __restrict__ inv,
                   float2* __restrict__ out, int64_t part_stride, int B, int Mc, int max_n, int Kb, int band_floats,
                   uint32_t tmem_cols, int* __restrict__ status, uint32_t wait_limit, int idle_mma) {
    using S = GfShape<T, false>;
    constexpr int NH = T * T;                       // complex entries of a tile
    constexpr int NR = 2 * NH;                      // real columns of D = rows of the B operand
    static_assert(NR == 32, "built for tile edge 4");
    constexpr uint32_t kABytes = 128 * 32 * 4;      // high (or low) part of one A chunk: 128 rows x 32 floats
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t empty_bar[2], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;

    const int G = (B + 31) >> 5;
    const int blk = blockIdx.x / G, g = blockIdx.x - blk * G;   // as in fused_gf_kernel: most expensive blocks first, groups together
    const int lt = blocks[4 * blk], q = blocks[4 * blk + 1];
    const int part = blocks[4 * blk + 2], parts = blocks[4 * blk + 3];
    const int nt = 2 * lt + 1, t_0 = q * T;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tau_t = P.tF[lt];
    // shared-memory carve: the two A buffers first (128-byte aligned), then as in the CUDA-core kernel
    unsigned char* a_st = smem_raw;                                                   // 2 x { high, low }
    float* b_hi = reinterpret_cast<float*>(a_st + 4 * kABytes);                       // [32][Kb] in MMA order
    float* b_lo = b_hi + NR * Kb;
    float2* acc = reinterpret_cast<float2*>(b_lo + NR * Kb);                          // [T][nt][32]
    float2* fo2 = acc + (size_t)T * max_n * 32;                                       // 2 x [n_o][T][32]
    float* band2 = reinterpret_cast<float*>(fo2 + (size_t)2 * T * max_n * 32);        // 2 x [n][n2]
    unsigned short* ulist = reinterpret_cast<unsigned short*>(band2 + 2 * band_floats);
    float2* H = reinterpret_cast<float2*>(reinterpret_cast<unsigned char*>(ulist) + ((kGfWarps * 4 * max_n + 15) & ~15));   // [Mc][NH][32]
    volatile int* failed = &failed_flag;

    if (threadIdx.x == 0) {
        mbar_init(&empty_bar[0], 1);
        mbar_init(&empty_bar[1], 1);
        mbar_init(&done_bar, 1);
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    for (int i = threadIdx.x; i < T * nt * 32; i += blockDim.x) acc[i] = make_float2(0.f, 0.f);
    int n_units = 0;   // this warp's phase-2 units, listed once per block
    for (int u = 0; u < gf_phase2_units<T, false, false>(nt); ++u)
        if (owner_tab[2 * lt * lt + u] == warp) {
            if (lane == 0) ulist[warp * 2 * max_n + n_units] = (unsigned short)u;
            ++n_units;
        }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const float2* slabF = SF + (int64_t)g * P.nSF * 32;
    const float2* slabG = SG + (int64_t)g * P.nSO * 32 + lane;

    auto stage_async = [&](const GfInfo& x, int buf) {
        const bool fst = x.role == 0;
        const int xn = 2 * x.l + 1, xn2 = 2 * x.l2 + 1, xno = fst ? xn2 : 2 * x.l1 + 1;
        const float4* src = reinterpret_cast<const float4*>(slabF + (int64_t)x.fo_off * 32);
        float4* dstf = reinterpret_cast<float4*>(fo2 + (size_t)buf * T * max_n * 32);
        for (int i = threadIdx.x; i < xno * T * 16; i += blockDim.x) __pipeline_memcpy_async(dstf + i, src + i, 16);
        float* dstb = band2 + buf * band_floats;
        for (int i = threadIdx.x; i < xn * xn2; i += blockDim.x) __pipeline_memcpy_async(dstb + i, P.cg + x.cgoff + i, 4);
        __pipeline_commit();
    };
    // weights of the entry: element i = (to, tile entry) -> conj(W)/std, zero outside the tile or beyond tau_out
    constexpr int kWtRegs = 2;
    auto wt_load = [&](const GfInfo& x, int i) -> float2 {
        const bool fst = x.role == 0;
        const int t = i / NH, idx = i - t * NH;
        const int i1 = idx / T, j1 = idx % T;
        const int a = fst ? i1 : j1, c = fst ? j1 : i1;   // owned / other channel inside their tiles
        const bool ok = t < x.to_n && (t_0 + a < tau_t) && (x.in0 + c < x.tau_o);
        const int t1 = fst ? t_0 + a : x.in0 + c, t2 = fst ? x.in0 + c : t_0 + a;
        const int ch = t1 * x.tau2 + t2;
        float2 w = make_float2(0.f, 0.f);
        if (ok) {
            w = __ldg(W + x.woff + (int64_t)t * x.tff + ch);
            const float sc = __ldg(inv + x.kglob + ch);
            w = make_float2(w.x * sc, -w.y * sc);
        }
        return w;
    };
    const int n_wt = (Kb / 2) * NH;   // every (to < Kb/2, entry): the padding is written as zeros each time
    auto wt_prefetch = [&](const GfInfo& x, float2 (&reg)[kWtRegs]) {
#pragma unroll
        for (int j = 0; j < kWtRegs; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_wt) reg[j] = wt_load(x, i);
        }
    };
    // B operand in the MMA's K-major core-matrix order: element (row n', column kk) at
    // (n'/8)*(Kb/4)*32 + (kk/4)*32 + (n'%8)*4 + kk%4 floats; rows (k, re), (k, im), columns (to, re), (to, im)
    auto b_put = [&](int i, float2 w) {
        const int t = i / NH, idx = i - t * NH;
        const int kk = 2 * t;
        const int r0 = 2 * idx, r1 = r0 + 1;
        const int o0 = (r0 >> 3) * (Kb / 4) * 32 + (kk >> 2) * 32 + (r0 & 7) * 4 + (kk & 3);
        const int o1 = (r1 >> 3) * (Kb / 4) * 32 + (kk >> 2) * 32 + (r1 & 7) * 4 + (kk & 3);
        const float hr = to_tf32(w.x), hi_ = to_tf32(w.y);
        // H.re = sum wr*gr - wi*gi,  H.im = sum wi*gr + wr*gi
        *reinterpret_cast<float2*>(b_hi + o0) = make_float2(hr, -hi_);
        *reinterpret_cast<float2*>(b_hi + o1) = make_float2(hi_, hr);
        *reinterpret_cast<float2*>(b_lo + o0) = make_float2(w.x - hr, -(w.y - hi_));
        *reinterpret_cast<float2*>(b_lo + o1) = make_float2(w.y - hi_, w.x - hr);
    };
    auto wt_store = [&](const GfInfo& x, const float2 (&reg)[kWtRegs]) {
#pragma unroll
        for (int j = 0; j < kWtRegs; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_wt) b_put(i, reg[j]);
        }
        for (int i = threadIdx.x + kWtRegs * blockDim.x; i < n_wt; i += blockDim.x) b_put(i, wt_load(x, i));
    };

    const int e_end = entry_begin[lt + 1];
    int e = entry_begin[lt] + part;
    GfInfo en;
    float2 wreg[kWtRegs];
    int buf = 0;
    int a_step = 0;      // A-buffer uses so far (all threads count alike)
    int n_entry = 0;     // entries whose MMAs were committed to done_bar: its phase parity
    bool ok = true;
    if (e < e_end) {
        en = entries[e];
        stage_async(en, 0);
        wt_prefetch(en, wreg);
    }
    const int mq = warp & 3, tq = warp >> 2;   // staging role: m inside the row tile, quarter of the chunk's 16 channels
    const uint32_t idesc = tc_idesc(128, NR);
    while (e < e_end) {
        const bool has_next = e + parts < e_end;
        GfInfo nxt;
        if (has_next) nxt = entries[e + parts];
        const int l = en.l, n = 2 * l + 1, n2 = 2 * en.l2 + 1;
        const int to_n = en.to_n;
        const bool first = en.role == 0;
        const float2* fo = fo2 + (size_t)buf * T * max_n * 32;
        const float* band = band2 + buf * band_floats;
        wt_store(en, wreg);          // the previous entry's MMAs are complete (its done barrier was waited for)
        __pipeline_wait_prior(0);
        __syncthreads();             // the previous entry's phase 2 is over: H and the idle staging halves are free
        if (has_next) stage_async(nxt, buf ^ 1);
        const float2* go = slabG + (int64_t)en.go_off * 32;
        const int lo_ = first ? en.l2 : en.l1;
        // ---- phase 1 on the tensor cores ----
        const int n_tiles = (n + 3) >> 2, n_kc = (2 * to_n + 31) >> 5;
        const int n_steps = n_tiles * n_kc;
        // the gO values of step s + 1 are loaded before step s is staged: the global-load latency of a step would
        // otherwise be paid once per step by all 16 warps together
        auto load_step = [&](int s_, float2 (&gv)[4]) {
            const int t = s_ / n_kc, kc = s_ - t * n_kc;
            const int mi = 4 * t + mq;
            const float2* gp = go + (((kc * 4 + tq) * n + min(mi, n - 1)) * T) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                gv[i] = (mi < n && kc * 16 + 4 * tq + i < to_n) ? gp[i * 32] : make_float2(0.f, 0.f);
        };
        float2 gv[4], gv_next[4];
        if (n_steps > 0) load_step(0, gv);
        for (int s_ = 0; s_ < n_steps; ++s_) {
            const int t = s_ / n_kc, kc = s_ - t * n_kc;
            if (s_ + 1 < n_steps) load_step(s_ + 1, gv_next);
            {
                const int ab = a_step & 1, use = a_step >> 1;
                if (use > 0) ok = mbar_wait_checked(&empty_bar[ab], (uint32_t)((use - 1) & 1), failed, wait_limit) && ok;
                const int mi = 4 * t + mq;
                if (mi < n) {
                    const int r = 32 * mq + lane;
                    float4* row_hi = reinterpret_cast<float4*>(a_st + (size_t)ab * 2 * kABytes) + (size_t)(r >> 3) * 64 + (r & 7);
                    float4* row_lo = row_hi + kABytes / 16;
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const float2 x0 = gv[2 * h2], x1 = gv[2 * h2 + 1];
                        float4 h, w;
                        h.x = to_tf32(x0.x); h.y = to_tf32(x0.y); h.z = to_tf32(x1.x); h.w = to_tf32(x1.y);
                        w.x = x0.x - h.x; w.y = x0.y - h.y; w.z = x1.x - h.z; w.w = x1.y - h.w;
                        row_hi[(2 * tq + h2) * 8] = h;
                        row_lo[(2 * tq + h2) * 8] = w;
                    }
                }
                fence_proxy_async();   // A chunk and (first step of the entry) the B operand become visible to the MMA
                tc_fence_before();
                __syncthreads();
                if (threadIdx.x == 0 && !idle_mma) {
                    if (ok && !*failed) {
                        tc_fence_after();
                        const uint32_t a_hi = smem_u32(a_st + (size_t)ab * 2 * kABytes), a_lo = a_hi + kABytes;
                        const uint32_t bh = smem_u32(b_hi) + kc * 1024, bl = smem_u32(b_lo) + kc * 1024;
                        const uint32_t b_sbo = (uint32_t)(Kb / 4) * 128;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t dah = smem_desc(a_hi + ks * 256, 128, 1024), dal = smem_desc(a_lo + ks * 256, 128, 1024);
                            const uint64_t dbh = smem_desc(bh + ks * 256, 128, b_sbo), dbl = smem_desc(bl + ks * 256, 128, b_sbo);
                            const uint32_t d = tmem_base + (uint32_t)t * NR;
                            tc_mma_tf32(d, dah, dbh, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
                            tc_mma_tf32(d, dal, dbh, idesc, 1u);
                            tc_mma_tf32(d, dah, dbl, idesc, 1u);
                        }
                    }
                    tc_commit(&empty_bar[ab]);
                    if (s_ == n_steps - 1) tc_commit(&done_bar);
                }
                ++a_step;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) gv[i] = gv_next[i];
        }
        if (n_tiles * n_kc > 0) {
            ok = mbar_wait_checked(&done_bar, (uint32_t)(n_entry & 1), failed, wait_limit) && ok;
            ++n_entry;   // phases of done_bar completed so far
        }
        tc_fence_after();
        // ---- H from tensor memory to the transit buffer, chunk by chunk, then phase 2 on the chunk ----
        for (int mc0 = 0; mc0 < n; mc0 += Mc) {
            const int mcn = min(Mc, n - mc0);
            if (mc0 > 0) __syncthreads();   // the previous chunk's readers are done with H
            {
                // this warp reads the rows with m % 4 == warp % 4; the four warps of a quadrant share its (m, half) pairs
                int m_first = mc0 + ((mq - mc0) & 3);
                int pair = 0;
                for (int mi = m_first; mi < mc0 + mcn; mi += 4)
                    for (int half = 0; half < 2; ++half, ++pair) {
                        if ((pair & 3) != tq) continue;   // warp-uniform
                        uint32_t rr[16];
                        if (ok && n_tiles * n_kc > 0) {
                            tmem_ld16(tmem_base + ((uint32_t)(32 * mq) << 16) + (uint32_t)((mi >> 2) * NR + half * 16), rr);
                        } else {   // an entry without work is zero; a block that gave up marks what it owns
#pragma unroll
                            for (int c = 0; c < 16; ++c) rr[c] = n_tiles * n_kc > 0 ? kNaNBits : 0u;
                        }
                        float2* h = H + ((size_t)(mi - mc0) * NH + half * 8) * 32 + lane;
#pragma unroll
                        for (int c = 0; c < 8; ++c) h[c * 32] = make_float2(__uint_as_float(rr[2 * c]), __uint_as_float(rr[2 * c + 1]));
                    }
            }
            tc_fence_before();
            __syncthreads();
            if (has_next && mc0 + Mc >= n) wt_prefetch(nxt, wreg);   // in flight during the last chunk's phase 2
            for (int k = 0; k < n_units; ++k) {
                const int u = ulist[warp * 2 * max_n + k];
                gf_phase2_unit<T, false, false>(u, first, H, fo, band, acc, lt, nt, l, lo_, en.l2, n2, mc0, mcn, lane);
            }
        }
        en = nxt;
        e += parts;
        buf ^= 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    float2* dst = out + (int64_t)part * part_stride;
    for (int i = threadIdx.x; i < T * nt * 32; i += blockDim.x) {
        const int ln = i & 31, rest = i >> 5;
        const int a = rest / nt, r = rest - a * nt;
        const int b = g * 32 + ln;
        if (b < B && t_0 + a < tau_t) dst[(int64_t)b * P.n_F + P.cumF[lt] + (int64_t)(t_0 + a) * nt + r] = acc[i];
    }
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
// Use the tensor-core forward?  Needs the plan's tables (tile edge 2 or 4, full product, tau_out <= 64) and pays off
// when the mixing dominates: measured on B200 against the CUDA-core forward (packing included) 1.25x faster at 12 and 16
// output channels, 2.2-2.7x at 32 and 64, 8 % slower at 8.  CGB200_OPT_TC_FWD overrides the default.
bool tc_wanted(const cgb200_plan* p) {
    if (!p->tc_ok) return false;
    if (p->opt[CGB200_OPT_TC_FWD] != CGB200_AUTO) return p->opt[CGB200_OPT_TC_FWD] == 1;
    return p->max_tau_out >= 12;
}

int64_t tc_pack_floats(const cgb200_plan* p) { return p->tc_ok ? p->tc_pack_off.back() : 0; }

// Splitting level of the tensor-core forward's contraction.  A block owns an SM (its pipeline stages fill the shared
// memory) and lasts in proportion to its cells, about 0.85 us each, so with few sample groups the degree with the most
// cells sets the kernel's duration: at lmax 14 with 16 channels and 64 samples there are 128 blocks for 148 SMs and the
// longest has 1024 of the 92 k cells.  The launch takes the coarsest level whose longest part is under a tenth of an
// SM's share of the cells (measured over lmax 10, 14, 20 with 16 to 64 channels and 32 to 256 samples: within 2 % of the
// best level everywhere; against no splitting 2.0x at lmax 10 with 64 channels and 64 samples, 1.2x at lmax 14 with 16
// channels and 64 samples, 1.07x at 256 samples), as long as the partial outputs stay under 256 MB.  The staged variant
// does not split.
int tc_fwd_level(const cgb200_plan* p, int64_t G) {
    if (!p->tc_ok) return 0;
    if (p->opt[CGB200_OPT_TC_STAGED] >= 1) return 0;
    if (p->opt[CGB200_OPT_TC_FWD_SPLIT] != CGB200_AUTO) return p->opt[CGB200_OPT_TC_FWD_SPLIT];
    const double share = (double)p->tc_total_cells * (double)G / std::max(p->num_sms, 1);
    const double out_bytes = (double)G * 32 * (double)p->d.n_O * sizeof(float2);
    int lv = 0;
    while (lv + 1 < cgb200_plan::kTcLevels && p->tc_longest[lv] > 0.1 * share &&
           p->tc_max_parts[lv + 1] * out_bytes <= 256.0 * (1 << 20))
        ++lv;
    return lv;
}

template <int T>
static int launch_tc(const cgb200_plan* p, int lv, const float2* SF, const float2* W, const float* inv, float* pack, float2* O,
                     float2* O_part, int B, int G, const float2* ff, cudaStream_t st) {
    constexpr int Kc = 2 * T * T;
    int n_max = 16;
    for (int v : p->tc_npad) n_max = std::max(n_max, v);
    if (p->tc_tiles[0].empty()) return CGB200_OK;
    if (W != nullptr) {   // null: `pack` already holds the packed weights (cgb200_layer_pack_weights)
        launch_begin(K_TC_PACK, st);
        if (p->d.n_cells > 0)
            tc_pack_kernel<T><<<p->d.n_cells, 256, 0, st>>>(p->d, p->d_tc_npad, p->d_tc_pack_off, W, inv, pack);
        launch_end(K_TC_PACK, st);
        CGB_CUDA(cudaGetLastError());
    }
    if (SF == nullptr) return CGB200_OK;   // packing only
    // flush groups: one per 64 accumulator columns; generator groups (= stages) take the warps that are left
    const int n_flush = n_max > 64 ? 2 : 1;
    const int s_cap = p->opt[CGB200_OPT_TC_STAGES] >= 2 ? std::min(kTcMaxStages - n_flush, p->opt[CGB200_OPT_TC_STAGES]) : kTcMaxStages - n_flush;
    const int idle = p->opt[CGB200_OPT_TEST_IDLE_MMA] == 1 ? 1 : 0;

    // Staged variant: a stage holds the A tile only; the ring takes what is left and must hold the largest cell (band rows,
    // the operand rows a row tile of four m can touch, the packed weights).  Preferred with room for two such cells.
    // Off unless asked for (CGB200_OPT_TC_STAGED 1: band rows, operand rows and weights staged; 2: band rows and weights only,
    // operands read through L1): measured on B200 within +-10 % of the kernel above at every shape tried (lmax 10 with 16,
    // 32, 64 channels, lmax 14 with 16, lmax 20 MST with 32), because both are bounded by the one thread that issues the
    // block's MMAs - about 65 cycles per tcgen05.mma, 12 per cell, each re-reading its 4 KB A tile from shared memory for
    // only 2 tau_out output columns - and, with the operand rows staged, by how few cells fit the ring.
    if (p->opt[CGB200_OPT_TC_STAGED] >= 1 && p->d_cg_pad != nullptr) {
        const bool stage_rows = p->opt[CGB200_OPT_TC_STAGED] == 1;
        size_t need_max = 0;
        for (const TripleRec& t : p->triples) {
            if (p->tO[t.l] == 0) continue;
            const int rows1 = stage_rows ? std::min(2 * t.l1 + 1, 2 * t.l2 + 1 + 3) : 0, rows2 = stage_rows ? 2 * t.l2 + 1 : 0;
            const size_t band = (size_t)((4 * ((2 * t.l2 + 4) & ~3) + 31) & ~31) * sizeof(float);
            need_max = std::max(need_max, band + (size_t)(rows1 + rows2) * T * 32 * sizeof(float2) + (size_t)2 * p->tc_npad[t.l] * Kc * sizeof(float));
        }
        const size_t a_bytes = (size_t)2 * 128 * Kc * sizeof(float);
        // A buffers: as many as leave a ring of two of the largest cells (at least one), at most kTcMaxStages
        int NA = 0;
        size_t ring = 0;
        const int na_cap = p->opt[CGB200_OPT_TC_ABUF] >= 2 ? std::min(kTcMaxStages, p->opt[CGB200_OPT_TC_ABUF]) : 4;
        for (int pass = 0; pass < 2 && NA == 0; ++pass)
            for (int cand = na_cap; cand >= 2; --cand) {
                if (cand * a_bytes >= kMaxDynSmem) continue;
                const size_t r = (kMaxDynSmem - cand * a_bytes) & ~(size_t)127;
                if (r >= (pass == 0 ? 2 * need_max : need_max + 128)) {
                    NA = cand;
                    ring = r;
                    break;
                }
            }
        const int S = std::min(s_cap, NA);   // generator groups (never more than A buffers: that combination ran into its bounded waits)
        if (NA >= 2) {
            const size_t smem = NA * a_bytes + ring;
            auto kern = fused_fwd_tc_staged_kernel<T>;
            CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            launch_begin(K_FWD_TC, st);
            kern<<<dim3((unsigned)p->tc_tiles[0].size() / 4, G), 32 * (4 * S + 2 + 4 * n_flush), smem, st>>>(p->d, p->d_tc_tiles[0], p->d_tc_npad, p->d_tc_pack_off, p->d_cg_pad,
                                                                            p->d_cell_cgpad, SF, pack, O, B, p->d_status, S, NA, n_flush, (int)ring,
                                                                            stage_rows ? 1 : 0, wait_polls(p), idle);
            launch_end(K_FWD_TC, st);
            CGB_CUDA(cudaGetLastError());
            return CGB200_OK;
        }
        set_error("tensor-core forward: a cell's operand rows and weights do not fit the shared-memory ring (lmax too large)");
        return CGB200_ERR_UNSUPPORTED;
    }
    const size_t stage_bytes = ((size_t)2 * 128 * Kc + (size_t)2 * n_max * Kc) * sizeof(float);
    const size_t cbuf_bytes = (size_t)(4 * kTcMaxStages + 1) * p->max_n * sizeof(float);
    const int n_stages = (int)std::min<size_t>(s_cap, (220 * 1024 - cbuf_bytes) / stage_bytes);
    const size_t smem = n_stages * stage_bytes + cbuf_bytes;
    if (n_stages < 2) {
        set_error("tensor-core forward: pipeline stages do not fit in shared memory");
        return CGB200_ERR_UNSUPPORTED;
    }
    const bool kept = T == 4 && ff != nullptr;
    auto kern = kept ? fused_fwd_tc_kernel<T, true> : fused_fwd_tc_kernel<T, false>;
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_begin(K_FWD_TC, st);
    const int64_t part_stride = (int64_t)B * p->d.n_O;
    kern<<<dim3((unsigned)p->tc_tiles[lv].size() / 4, G), 32 * (4 * n_stages + 1 + 4 * n_flush), smem, st>>>(
        p->d, p->d_tc_tiles[lv], p->d_tc_npad, p->d_tc_pack_off, SF, pack, O, O_part, part_stride, B, n_max, p->max_n, p->d_status,
        n_stages, n_flush, wait_polls(p), idle, kept ? ff : nullptr, gff_group_elems(p), p->d_gff_off);
    launch_end(K_FWD_TC, st);
    CGB_CUDA(cudaGetLastError());
    if (p->tc_max_parts[lv] > 1) {
        launch_parts_reduce(K_FWD_REDUCE, p->d.cumO, p->d.lmax + 1, p->d.n_O, p->d_tc_parts[lv], O_part, part_stride, O, B, true, st);
        CGB_CUDA(cudaGetLastError());
    }
    return CGB200_OK;
}

int launch_fwd_tc(const cgb200_plan* p, int lv, const float2* SF, const float2* W, const float* inv, float* pack, float2* O,
                  float2* O_part, int B, int G, const float2* ff, cudaStream_t st) {
    if (p->d.tile == 4) return launch_tc<4>(p, lv, SF, W, inv, pack, O, O_part, B, G, ff, st);
    if (p->d.tile == 2) return launch_tc<2>(p, lv, SF, W, inv, pack, O, O_part, B, G, nullptr, st);
    set_error("internal: tensor-core forward asked for an unsupported tile edge");
    return CGB200_ERR_UNSUPPORTED;
}


// Weight gradient on the tensor cores: tile edge 4, full product, where the forward's tables exist.  Same default
// threshold as the forward (16 output channels); CGB200_OPT_TC_GRAD_W overrides it.
bool tc_gw_wanted(const cgb200_plan* p) {
    if (!p->tc_gw_ok || p->tc_gw_tiles.empty()) return false;
    if (p->opt[CGB200_OPT_TC_GRAD_W] != CGB200_AUTO) return p->opt[CGB200_OPT_TC_GRAD_W] == 1;
    // tile edge 4: faster than the CUDA-core kernel at every width measured (2x at 8 output channels, 2.9x at 12, 3.3x at
    // 16, 5-8x at 32 and 64).  Tile edge 5 is built and tested but stays off by default: at 5 channels (lmax 10, batch
    // 100) it takes 126 us against 98 us - blocks of two cells with at most 21 chunks each spend their time filling and
    // draining the pipeline
    return p->d.tile == 4;
}

template <int T>
static int launch_gw_tc_t(const cgb200_plan* p, const float2* SF, const float2* SG, const float* inv, float2* gW, float2* gw_part,
                          int max_slices, int G, const float2* ff, cudaStream_t st) {
    int n_max = 16;
    for (int v : p->tc_npad) n_max = std::max(n_max, v);
    const int n_tiles = (int)p->tc_gw_tiles.size() / 2;
    if (n_tiles == 0) return CGB200_OK;
    const size_t stage_bytes = (size_t)2 * 16 * kGwSbo + (size_t)2 * (n_max / 8) * kGwSbo;
    const size_t cbuf_bytes = (size_t)(4 * kTcMaxStages + 1) * p->max_n * sizeof(float);
    const int n_flush = n_max > 64 ? 2 : 1;   // flush groups: one per 64 accumulator columns
    int n_stages = (int)std::min<size_t>(kTcMaxStages - n_flush, (kMaxDynSmem - cbuf_bytes) / stage_bytes);
    if (p->opt[CGB200_OPT_TC_STAGES] >= 2) n_stages = std::min(n_stages, p->opt[CGB200_OPT_TC_STAGES]);
    if (n_stages < 2) {
        set_error("tensor-core weight gradient: pipeline stages do not fit in shared memory");
        return CGB200_ERR_UNSUPPORTED;
    }
    // with few blocks (few cells) the sample groups are sliced over several blocks and the partial sums reduced in order
    int slices = (int)std::min<int64_t>(std::min(max_slices, G), (4 * (int64_t)p->num_sms + n_tiles - 1) / n_tiles);
    slices = std::max(1, std::min(slices, 65535));
    if (gw_part == nullptr) slices = 1;
    const size_t smem = n_stages * stage_bytes + cbuf_bytes;
    const bool kept = T == 4 && p->gff_ok && ff != nullptr;
    auto kern = kept ? fused_gw_tc_kernel<T, true> : fused_gw_tc_kernel<T, false>;
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_begin(K_GW_TC, st);
    kern<<<dim3(n_tiles, slices), 32 * (4 * n_stages + 1 + 4 * n_flush), smem, st>>>(p->d, p->d_tc_gw_tiles, p->d_tc_npad, SF, SG, inv,
                                                                       slices > 1 ? gw_part : gW, G, n_max, p->max_n, p->d_status,
                                                                       n_stages, n_flush, p->d.w_len, wait_polls(p),
                                                                       p->opt[CGB200_OPT_TEST_IDLE_MMA] == 1 ? 1 : 0,
                                                                       kept ? ff : nullptr, gff_group_elems(p), p->d_gff_off);
    launch_end(K_GW_TC, st);
    CGB_CUDA(cudaGetLastError());
    if (slices > 1) {
        launch_gw_reduce(p, gw_part, slices, gW, st);
        CGB_CUDA(cudaGetLastError());
    }
    return CGB200_OK;
}

int launch_gw_tc(const cgb200_plan* p, const float2* SF, const float2* SG, const float* inv, float2* gW, float2* gw_part,
                 int max_slices, int G, const float2* ff, cudaStream_t st) {
    if (p->d.tile == 4) return launch_gw_tc_t<4>(p, SF, SG, inv, gW, gw_part, max_slices, G, ff, st);
    if (p->d.tile == 5) return launch_gw_tc_t<5>(p, SF, SG, inv, gW, gw_part, max_slices, G, nullptr, st);
    set_error("internal: tensor-core weight gradient asked for an unsupported tile edge");
    return CGB200_ERR_UNSUPPORTED;
}

// Input gradient with phase 1 on the tensor cores: tile edge 4, full product, 2 lmax + 1 <= 64 (the gFF tile of an entry
// must fit the 512 columns of tensor memory).  Off unless CGB200_OPT_TC_GRAD_F is 1: measured on B200 it matches but does not beat
// the CUDA-core kernel (lmax 14, 16 channels, batch 64: 8.5 against 7.5 ms; lmax 10, 64 channels: 62 against 59 ms).
// Every (row tile, 16-channel chunk) step moves a 32 KB A chunk through one of two shared-memory buffers, so a step
// lasts half the issue-to-completion latency of its MMAs (about 1 us per step); a deeper ring does not fit beside the
// phase-2 buffers, and a wider N per step (several cells per MMA) needs more than the 512 columns of tensor memory.
bool tc_gf_wanted(const cgb200_plan* p) {
    if (!p->tc_ok || p->d.tile != 4 || p->max_n > 64) return false;
    return p->opt[CGB200_OPT_TC_GRAD_F] == 1;
}

int launch_gf_tc(const cgb200_plan* p, int lv, const float2* SF, const float2* SG, const float2* W, const float* inv, float2* out,
                 int64_t part_stride, int B, int G, cudaStream_t st) {
    constexpr int T = 4, NH = 16;
    const int nblk = (int)p->gf2_blocks[lv].size() / 4;
    if (nblk == 0) return CGB200_OK;
    const int Kb = ((2 * std::max(p->max_tau_out, 1) + 31) / 32) * 32;
    const int band_floats = (int)(p->gen_band_bytes / sizeof(float));
    const size_t fixed = (size_t)4 * 128 * 32 * 4 + (size_t)2 * 32 * Kb * 4 + (size_t)3 * T * p->max_n * 32 * sizeof(float2) +
                         2 * p->gen_band_bytes + (size_t)((kGfWarps * 4 * p->max_n + 15) & ~15);
    const size_t per_m = (size_t)NH * 32 * sizeof(float2);
    const size_t budget = kMaxDynSmem;
    if (fixed + 4 * per_m > budget) {
        set_error("tensor-core input gradient: staging areas do not fit in shared memory");
        return CGB200_ERR_UNSUPPORTED;
    }
    const int Mc = (int)std::min<size_t>(p->max_n, (budget - fixed) / per_m);
    const size_t smem = fixed + (size_t)Mc * per_m;
    uint32_t cols = 32;
    while (cols < (uint32_t)(32 * ((p->max_n + 3) / 4))) cols <<= 1;
    auto kern = fused_gf_tc_kernel<T>;
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_begin(K_GF_TC, st);
    kern<<<(unsigned)((int64_t)nblk * G), kGfWarps * 32, smem, st>>>(p->d, p->d_gf_info, p->d_gf_begin, p->d_gf2_blocks[lv], p->d_gf_owner, SF, SG, W, inv,
                                                     out, part_stride, B, Mc, p->max_n, Kb, band_floats, cols, p->d_status,
                                                     wait_polls(p), p->opt[CGB200_OPT_TEST_IDLE_MMA] == 1 ? 1 : 0);
    launch_end(K_GF_TC, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // namespace cgb200
