// Spherical-harmonic projection of sampled functions: the step in front of the CG network.
//
//   coefs[r, c] = scale * sum_p f[r, p] * M[p, c]          r: function (sample x channel), p: sample point, c: (l, m)
//
// with M the complex basis the host prepared (quadrature weight times conj(Y_lm) for a grid transform, Y_lm itself for
// scattered points) and scale = 4 pi / P.  This is the contraction of the reference's `get_sph_coefs`
// (utils/s2_sph.py:79-86: `(fs * ws)[:, None] * conj(sphs)).mean(0) * 4 pi`) and `get_coef_C`
// (utils/geometries.py:125-144: `(f[:, None] * sph).mean(0) * 4 pi`), which numpy evaluates one function at a time; here
// all functions of a batch go through one real GEMM  [rows x P] x [P x 2 n_cols]  on the tensor cores:
// tcgen05.mma kind::tf32 with the 3xTF32 split (A = Ah + Al, B = Bh + Bl, D += Ah Bh + Al Bh + Ah Bl), accumulator in
// tensor memory, both operands pre-packed in the MMA's shared-memory order and brought in by cp.async.bulk, so the main
// kernel has no generator warps: one lane issues copies, one lane issues MMAs, four warps keep rounded running sums (the
// tensor core adds with truncation, so the contraction is summed in pieces of kChunkSteps steps) and write the result.
#include <algorithm>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cgb200 {

constexpr int kShKc = 32;                 // K extent of a chunk (sample points)
constexpr int kShTileFloats = 128 * kShKc;   // one 128-row operand tile of a chunk, high or low part
constexpr int kShMaxStages = 4;
constexpr int kShThreads = 192;           // copy warp, MMA warp, four flush warps

// element (row r, column k) of a [rows x 32] K-major tile in 8-row x 16-byte core matrices
__host__ __device__ inline int sh_core_off(int r, int k) { return (r >> 3) * 256 + (k >> 2) * 32 + (r & 7) * 4 + (k & 3); }

// f[rows][P] -> per (row tile, chunk) a block { high [128 x 32], low [128 x 32] }; rows and points beyond the end are zero
__global__ void __launch_bounds__(256)
sh_pack_rows_kernel(const float* __restrict__ f, int64_t rows, int64_t P, int n_chunks, float* __restrict__ out) {
    const int64_t tile = blockIdx.y;
    const int q = blockIdx.x;
    float* hi = out + (tile * n_chunks + q) * 2 * kShTileFloats;
    float* lo = hi + kShTileFloats;
    for (int e = threadIdx.x; e < kShTileFloats; e += blockDim.x) {
        const int r = e >> 5, k = e & 31;   // consecutive threads read consecutive points of a row
        const int64_t row = tile * 128 + r, p = (int64_t)q * kShKc + k;
        const float v = (row < rows && p < P) ? f[row * P + p] : 0.f;
        const float h = to_tf32(v);
        const int off = sh_core_off(r, k);
        hi[off] = h;
        lo[off] = v - h;
    }
}

// basis[P][n_cols] complex -> per (column tile, chunk) a block { high [nt x 32], low [nt x 32] } of the real form:
// real column 2c = Re M[., c], 2c + 1 = Im M[., c]
__global__ void __launch_bounds__(256)
sh_pack_basis_kernel(const float2* __restrict__ basis, int64_t P, int n_cols, int nt, int n_chunks, float* __restrict__ out) {
    const int ct = blockIdx.y, q = blockIdx.x;
    float* hi = out + ((int64_t)ct * n_chunks + q) * 2 * nt * kShKc;
    float* lo = hi + nt * kShKc;
    for (int e = threadIdx.x; e < nt * kShKc; e += blockDim.x) {
        const int k = e / nt, np = e - k * nt;   // consecutive threads read consecutive columns of a point
        const int64_t p = (int64_t)q * kShKc + k;
        const int col = ct * nt + np, c = col >> 1;
        float v = 0.f;
        if (p < P && c < n_cols) {
            const float2 z = basis[p * n_cols + c];
            v = (col & 1) ? z.y : z.x;
        }
        const float h = to_tf32(v);
        const int off = sh_core_off(np, k);
        hi[off] = h;
        lo[off] = v - h;
    }
}

// grid = (row tiles, column tiles)
__global__ void __launch_bounds__(kShThreads)
sh_project_kernel(const float* __restrict__ rows_packed, const float* __restrict__ basis_packed, float2* __restrict__ coefs,
                  int64_t rows, int n_cols, int nt, int n_chunks, int n_stages, float scale, int* __restrict__ status,
                  uint32_t wait_limit) {
    constexpr int kFlushChunks = kChunkSteps / 12;   // chunks (4 K steps x 3 MMAs) summed in tensor memory before a flush
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kShMaxStages], empty_bar[kShMaxStages], chunk_full[2], chunk_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rt = blockIdx.x;
    const int ct = blockIdx.y;
    const uint32_t a_bytes = 2 * kShTileFloats * sizeof(float), b_bytes = (uint32_t)(2 * nt * kShKc * sizeof(float));
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t tmem_cols = 2 * nt <= 32 ? 32u : 2 * nt <= 64 ? 64u : 2 * nt <= 128 ? 128u : 256u;   // two regions of nt columns
    volatile int* failed = &failed_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int r = 0; r < 2; ++r) {
            mbar_init(&chunk_full[r], 1);
            mbar_init(&chunk_free[r], 4);
        }
        failed_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------- copies: chunk q of both operands -> stage q % S ----------------
        if (lane == 0) {
            const float* a_src = rows_packed + rt * n_chunks * 2 * kShTileFloats;
            const float* b_src = basis_packed + (int64_t)ct * n_chunks * 2 * nt * kShKc;
            bool ok = true;
            int last = -1;
            for (int q = 0; q < n_chunks && ok; ++q) {
                const int s = q % n_stages, u = q / n_stages;
                if (u > 0) ok = mbar_wait(&empty_bar[s], (uint32_t)((u - 1) & 1), failed, wait_limit);
                if (!ok) break;
                unsigned char* st = smem_raw + (size_t)s * stage_bytes;
                mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
                bulk_g2s(st, a_src + (int64_t)q * 2 * kShTileFloats, a_bytes, &full_bar[s]);
                bulk_g2s(st + a_bytes, b_src + (int64_t)q * 2 * nt * kShKc, b_bytes, &full_bar[s]);
                last = q;
            }
            // a block that gave up may leave before its newest copies were consumed: let them land first
            if (!ok || *failed)
                for (int q = max(0, last - n_stages + 1); q <= last; ++q) mbar_drain(&full_bar[q % n_stages], (uint32_t)((q / n_stages) & 1), wait_limit);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(128, nt);
            bool ok = true;
            for (int q = 0; q < n_chunks && ok; ++q) {
                const int s = q % n_stages, u = q / n_stages;
                const int j = q / kFlushChunks, r = j & 1;
                const bool first = q - j * kFlushChunks == 0;
                if (first && j >= 2) ok = mbar_wait(&chunk_free[r], (uint32_t)(((j >> 1) - 1) & 1), failed, wait_limit);
                if (!ok) break;
                ok = mbar_wait(&full_bar[s], (uint32_t)(u & 1), failed, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(r * nt);
                const uint32_t a_hi = smem_u32(smem_raw + (size_t)s * stage_bytes);
                const uint32_t a_lo = a_hi + kShTileFloats * 4;
                const uint32_t b_hi = a_hi + a_bytes;
                const uint32_t b_lo = b_hi + (uint32_t)nt * kShKc * 4;
                const uint64_t dah0 = smem_desc(a_hi, 128, 1024), dal0 = smem_desc(a_lo, 128, 1024);
                const uint64_t dbh0 = smem_desc(b_hi, 128, 1024), dbl0 = smem_desc(b_lo, 128, 1024);
#pragma unroll
                for (int ks = 0; ks < kShKc / 8; ++ks) {
                    const uint64_t dah = desc_advance(dah0, ks * 256), dal = desc_advance(dal0, ks * 256);
                    const uint64_t dbh = desc_advance(dbh0, ks * 256), dbl = desc_advance(dbl0, ks * 256);
                    tc_mma_tf32(d, dah, dbh, idesc, (!first || ks > 0) ? 1u : 0u);
                    tc_mma_tf32(d, dal, dbh, idesc, 1u);
                    tc_mma_tf32(d, dah, dbl, idesc, 1u);
                }
                tc_commit(&empty_bar[s]);
                if (q - j * kFlushChunks == kFlushChunks - 1 || q == n_chunks - 1) tc_commit(&chunk_full[r]);
            }
        }
    } else {
        // ---------------- flush warps: rounded running sums, then the coefficients ----------------
        const int wq = warp & 3;   // the TMEM lane quarter this warp may read
        const int n_flushes = (n_chunks + kFlushChunks - 1) / kFlushChunks;
        float run[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) run[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_flushes && ok; ++j) {
            const int r = j & 1;
            ok = mbar_wait_warp(&chunk_full[r], (uint32_t)((j >> 1) & 1), failed, wait_limit);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                if (16 * c8 < nt) {   // warp-uniform
                    uint32_t rr[16];
                    tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(r * nt + 16 * c8), rr);
#pragma unroll
                    for (int i = 0; i < 16; ++i) run[16 * c8 + i] += __uint_as_float(rr[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&chunk_free[r]);
        }
        const int64_t row = rt * 128 + wq * 32 + lane;
        if (row < rows) {
            float2* out = coefs + row * n_cols;
            const float nanv = __uint_as_float(kNaNBits);   // a block that gave up marks the outputs it owns
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int c = (ct * nt + 16 * c8) / 2 + i;
                    if (16 * c8 < nt && c < n_cols)
                        out[c] = ok ? make_float2(run[16 * c8 + 2 * i] * scale, run[16 * c8 + 2 * i + 1] * scale) : make_float2(nanv, nanv);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
    if (threadIdx.x == 0 && failed_flag) atomicExch(status, 1);
}

// width of a column tile: all 2 n_cols real columns rounded up to 16 when they fit 128, else 128
static int sh_tile_cols(int n_cols) { return std::min(128, ((2 * n_cols + 15) / 16) * 16); }
static int sh_col_tiles(int n_cols) { return (2 * n_cols + sh_tile_cols(n_cols) - 1) / sh_tile_cols(n_cols); }
static int sh_chunks(int64_t P) { return (int)((P + kShKc - 1) / kShKc); }

}  // namespace cgb200

using namespace cgb200;

extern "C" {

int64_t cgb200_sh_basis_bytes(int64_t n_points, int n_cols) {
    if (n_points <= 0 || n_cols <= 0 || n_points > (1ll << 30)) {
        set_error("cgb200_sh_basis_bytes: sizes out of range");
        return -1;
    }
    return (int64_t)sh_col_tiles(n_cols) * sh_chunks(n_points) * 2 * sh_tile_cols(n_cols) * kShKc * (int64_t)sizeof(float);
}

int64_t cgb200_sh_workspace_bytes(int64_t rows, int64_t n_points) {
    if (rows < 0 || n_points <= 0 || n_points > (1ll << 30)) {
        set_error("cgb200_sh_workspace_bytes: sizes out of range");
        return -1;
    }
    return 256 + ((rows + 127) / 128) * sh_chunks(n_points) * 2 * kShTileFloats * (int64_t)sizeof(float);
}

int cgb200_sh_basis_pack(const float* basis, int64_t n_points, int n_cols, float* packed, void* stream) {
    CGB_REQUIRE(basis != nullptr && packed != nullptr, "null buffer");
    CGB_REQUIRE(n_points > 0 && n_points <= (1ll << 30) && n_cols > 0 && n_cols <= (1 << 20), "sizes out of range");
    CGB_REQUIRE((reinterpret_cast<uintptr_t>(basis) & 7) == 0 && (reinterpret_cast<uintptr_t>(packed) & 255) == 0,
                "basis must be 8-byte aligned and the packed buffer 256-byte aligned");
    const int nt = sh_tile_cols(n_cols), nct = sh_col_tiles(n_cols), nq = sh_chunks(n_points);
    cudaStream_t st = (cudaStream_t)stream;
    launch_begin(K_SH_PACK, st);
    sh_pack_basis_kernel<<<dim3(nq, nct), 256, 0, st>>>((const float2*)basis, n_points, n_cols, nt, nq, packed);
    launch_end(K_SH_PACK, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

int cgb200_sh_project(const float* f, int64_t rows, int64_t n_points, int n_cols, const float* basis_packed, float scale,
                      float* coefs, void* workspace, int64_t workspace_bytes, int32_t* status_word, void* stream) {
    CGB_REQUIRE(rows >= 0 && n_points > 0 && n_points <= (1ll << 30) && n_cols > 0 && n_cols <= (1 << 20), "sizes out of range");
    if (rows == 0) return CGB200_OK;
    CGB_REQUIRE(f != nullptr && basis_packed != nullptr && coefs != nullptr && status_word != nullptr, "null buffer");
    CGB_REQUIRE((reinterpret_cast<uintptr_t>(coefs) & 7) == 0 && (reinterpret_cast<uintptr_t>(basis_packed) & 255) == 0,
                "coefs must be 8-byte aligned and the packed basis 256-byte aligned");
    const int64_t need = cgb200_sh_workspace_bytes(rows, n_points);
    if (workspace == nullptr || workspace_bytes < need) {
        set_error("workspace too small: need " + std::to_string(need) + " bytes");
        return CGB200_ERR_WORKSPACE;
    }
    CGB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
    const int nt = sh_tile_cols(n_cols), nct = sh_col_tiles(n_cols), nq = sh_chunks(n_points);
    const int64_t row_tiles = (rows + 127) / 128;
    CGB_REQUIRE(row_tiles <= 0x7fffffff && nq <= 65535 && nct <= 65535, "too many tiles for one launch");
    cudaStream_t st = (cudaStream_t)stream;
    float* rows_packed = (float*)workspace;
    launch_begin(K_SH_PACK, st);
    // grid.y is limited to 65535 row tiles per launch
    for (int64_t t0 = 0; t0 < row_tiles; t0 += 65535) {
        const int64_t nty = std::min<int64_t>(65535, row_tiles - t0);
        sh_pack_rows_kernel<<<dim3(nq, (unsigned)nty), 256, 0, st>>>(f + t0 * 128 * n_points, rows - t0 * 128, n_points, nq,
                                                                   rows_packed + t0 * nq * 2 * kShTileFloats);
    }
    launch_end(K_SH_PACK, st);
    CGB_CUDA(cudaGetLastError());
    const size_t stage_bytes = (size_t)2 * kShTileFloats * sizeof(float) + (size_t)2 * nt * kShKc * sizeof(float);
    const int n_stages = (int)std::min<size_t>(kShMaxStages, kMaxDynSmem / stage_bytes);
    const size_t smem = n_stages * stage_bytes;
    auto kern = sh_project_kernel;
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_begin(K_SH_PROJECT, st);
    kern<<<dim3((unsigned)row_tiles, nct), kShThreads, smem, st>>>(rows_packed, basis_packed, (float2*)coefs, rows, n_cols, nt, nq, n_stages,
                                                                 scale, status_word, kDefaultWaitPolls);
    launch_end(K_SH_PROJECT, st);
    CGB_CUDA(cudaGetLastError());
    return CGB200_OK;
}

}  // extern "C"
