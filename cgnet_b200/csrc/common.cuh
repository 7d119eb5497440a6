// Shared definitions of libcgnet_b200: plan tables as the kernels see them, error plumbing, and the register-tiled
// generator of CG-product values that every kernel touching the product is built from.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <mutex>
#include <vector>

#include "../../include/cgnet_b200.h"

namespace cgb200 {

constexpr int kMaxLmax = 511;        // same ceiling the reference asserts (cudaCG_sparse.cu:23)
// Dynamic shared memory a launch may ask for: the 227 KB a block can own less 1 KB for the kernels' static __shared__
// variables (barriers, counters, reduction scratch), which count against the same limit.
constexpr size_t kMaxDynSmem = 226 * 1024;
constexpr size_t kSmemPerSM = 228 * 1024;   // shared memory of an SM; every resident block reserves 1 KB of it
constexpr int kMaxTile = 6;          // largest channel-tile edge the register-tiled kernels are instantiated for

// One admissible (l, l1, l2) triple with everything a kernel needs to find its operands and its outputs.
struct TripleRec {
    int l, l1, l2;
    int tau1, tau2;       // channel counts of the two operand fragments
    int nch;              // mid channels this triple produces: tau1*tau2 (tau1 in depthwise mode)
    int toff;             // first mid channel of the triple inside degree l
    int kglob;            // the same, counted over all degrees (index into stds)
    int f1off, f2off;     // start of fragment l1 / l2 inside one sample of F, in complex elements
    int cgoff;            // start of the triple's band table, in floats (tables beyond 2^31 floats are rejected)
    int nt1, nt2;         // channel tiles along t1 and t2 (tile edge = Plan::tile)
    int cell0;            // index of the triple's first cell
    int64_t ffoff;        // start of the triple's block inside one sample of FF, in complex elements
    int64_t woff;         // column of the triple inside W_l: cumW[l] + toff (row stride t_FF[l]), complex elements
};

// A cell = one (tile of t1) x (tile of t2) block of one triple: the unit of work a thread computes for one (b, m).
struct CellRec {
    int triple;
    short t1_0, t2_0;
};

// Everything a fused kernel needs about one cell in a single 32-byte record (one uniform load instead of a chain of
// dependent ones through CellRec and TripleRec).
struct CellInfo {
    int cgoff;        // band table of the triple
    int o1, o2;       // slab offsets (in elements of 32 lanes) of the t1 tile / t2 tile at m index 0
    int wch0;         // toff + first mid channel of the cell: column inside W_l
    int kch0;         // kglob + first mid channel of the cell: index into stds / inv
    int tau2;         // channel (t1_0+i, t2_0+j) of the cell is wch0 + i*tau2 + j   (depthwise: wch0 + i)
    short l1, l2;
    short v1, v2;     // valid channels of the tile along t1 / t2
};

// One warp-task of the fused weight-gradient kernel.
struct GwTask {
    int triple;
    short q1, gi;     // t1 tile and first row of the task inside it
    short q2, qo;     // t2 tile, tau_out tile
    short ni, pad_;   // rows of t1 the task covers
};
// Rows of t1 per weight-gradient task, by tile edge: a tile is cut into groups of A rows and, where A does not divide
// the edge, one last group of B rows (tile edge 5 = 2 + 2 + 1), so that no task carries a masked row.  Two rows keep
// the kernel under 168 registers with its operand prefetch, i.e. three blocks per SM; groups of three rows need 254.
template <int T>
struct GwRows {
    static constexpr int A = T == 1 ? 1 : T == 2 ? 2 : T == 3 ? 3 : T == 4 ? 2 : T == 5 ? 2 : 1;
    static constexpr int B = T % A;
};
inline int gw_rows_a(int T) { return T == 1 ? 1 : T == 2 ? 2 : T == 3 ? 3 : T == 4 ? 2 : T == 5 ? 2 : 1; }

// One entry of the fused input-gradient kernel with its triple's data inlined.
struct GfInfo {
    int cgoff;
    int go_off;       // cumSO[l]: slab offset of the output-gradient fragment
    int fo_off;       // slab offset of the other operand's tile (depthwise: of the other operand's fragment)
    int kglob;
    int tau2, tff, to_n;
    int tau_o;        // channels of the other operand
    short l, l1, l2;
    short role;       // 0: the owned fragment is the first operand, 1: the second
    short in0;        // first channel of the other operand's tile
    short pad_;
    int cell0;        // first cell of the triple: cell (tile i of t1, tile j of t2) is cell0 + i * ceil(tau2 / T) + j
    int pad2_;
    int64_t woff;     // cumW[l] + toff
};

// Work item of the forward product kernel: a run of cells of one triple with ncell * (2l+1) <= kGenThreads.
struct GenItem {
    int triple;
    int cell0;   // first cell (absolute index)
    int ncell;
};
constexpr int kGenThreads = 256;
constexpr int kGfWarps = 16;   // warps of an input-gradient block (the plan's phase-2 unit assignment is made for this count)

// Work entry of the fused input-gradient kernel: one triple in which a given fragment takes part, the role it plays
// there (0: first operand, 1: second operand) and the first channel of the tile of the *other* operand.
struct GfEntry {
    int triple;
    short role;
    short in0;
};

// Plan tables in device memory.
struct PlanDev {
    int lmax;
    int tile;
    int depthwise;
    int n_triples;
    int n_cells;
    int has_out;
    int64_t n_F, n_FF, n_O, w_len;
    int sum_tff;
    const TripleRec* triples;
    const CellRec* cells;
    const CellInfo* cell_info;
    const int* cell_begin;       // [lmax+2]  cells of degree l are cell_begin[l] .. cell_begin[l+1]
    const int* triple_begin;     // [lmax+2]
    const int* tF;               // [lmax+1]
    const int* tO;               // [lmax+1]
    const int* tFF;              // [lmax+1]
    const int64_t* cumF;         // [lmax+2] complex elements
    const int64_t* cumFF;
    const int64_t* cumO;
    const int64_t* cumW;
    const int* cumT;             // [lmax+2] running sum of tFF
    // "slab" layout of an activation for the fused kernels: samples in groups of 32 (one per lane), inside a group
    // fragment l starts at cumS[l] and holds its channels in tiles of `tile`: element (t, m) sits at
    // ((t/tile * (2l+1) + m+l) * tile + t%tile); channels beyond tau_l are zero.  One element = 32 lanes of float2.
    const int* cumSF;            // [lmax+2] input activation
    const int* cumSO;            // [lmax+2] output activation
    int nSF, nSO;
    const int* role1_begin;      // [lmax+2] triples whose first operand is fragment l
    const int* role1_list;
    const int* role2_begin;      // [lmax+2] triples whose second operand is fragment l
    const int* role2_list;
    const float* cg;
};

void set_error(const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

// Kernel identifiers for launch accounting and the optional per-kernel CUDA-event timing (cgb200_timing_*).
enum KernelId {
    K_CG_TABLE = 0, K_CG_FWD, K_CG_BWD, K_FN_STATS, K_WMM_FWD, K_WMM_BWD_W, K_WMM_BWD_MID,
    K_PREP, K_STATS, K_FWD, K_GW, K_GF, K_GF_REDUCE, K_GW_REDUCE, K_TC_PACK, K_FWD_TC, K_GW_TC, K_GF_TC, K_SH_PACK, K_SH_PROJECT,
    K_RAY_PACK, K_RAY_CAST, K_FWD_REDUCE, K_GFF_PACK, K_GFF_GEMM, K_COUNT
};
// Bracket every kernel launch with these: they count the launch and, while timing is enabled, record a CUDA event on
// the launching stream before and after it.
void launch_begin(int kid, cudaStream_t st);
void launch_end(int kid, cudaStream_t st);
bool timing_active();   // per-kernel event timing is on (cgb200_timing_enable)

#define CGB_CUDA(call)                                         \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call);  \
    } while (0)

#define CGB_REQUIRE(cond, msg)                  \
    do {                                        \
        if (!(cond)) {                          \
            set_error(msg);                     \
            return CGB200_ERR_ARGUMENT;         \
        }                                       \
    } while (0)

}  // namespace cgb200

// Run a statement with TT / DD bound to the plan's tile edge and depthwise flag as compile-time constants.
#define CGB_DISPATCH_TILE(T_, DW_, ...)                                          \
    switch ((T_) * 2 + ((DW_) ? 1 : 0)) {                                        \
        case 2: { constexpr int TT = 1; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        case 3: { constexpr int TT = 1; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }    \
        case 4: { constexpr int TT = 2; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        case 5: { constexpr int TT = 2; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }    \
        case 6: { constexpr int TT = 3; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        case 7: { constexpr int TT = 3; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }    \
        case 8: { constexpr int TT = 4; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        case 9: { constexpr int TT = 4; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }    \
        case 10: { constexpr int TT = 5; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }  \
        case 11: { constexpr int TT = 5; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        case 12: { constexpr int TT = 6; constexpr bool DD = false; (void)TT; (void)DD; __VA_ARGS__; break; }  \
        case 13: { constexpr int TT = 6; constexpr bool DD = true; (void)TT; (void)DD; __VA_ARGS__; break; }   \
        default: cgb200::set_error("internal: tile edge out of range"); return CGB200_ERR_UNSUPPORTED;  \
    }

// tensor-core forward (fused_tc.cu)
struct cgb200_plan;
namespace cgb200 {
constexpr uint32_t kDefaultWaitPolls = 4000000;   // polls of mbarrier.try_wait before a bounded wait gives up
inline uint32_t wait_polls(const cgb200_plan* p);
bool tc_wanted(const cgb200_plan* p);
bool tc_gw_wanted(const cgb200_plan* p);
bool tc_gf_wanted(const cgb200_plan* p);
int launch_gf_tc(const cgb200_plan* p, int lv, const float2* SF, const float2* SG, const float2* W, const float* inv, float2* out,
                 int64_t part_stride, int B, int G, cudaStream_t st);
int launch_gw_tc(const cgb200_plan* p, const float2* SF, const float2* SG, const float* inv, float2* gW, float2* gw_part,
                 int max_slices, int G, const float2* ff, cudaStream_t st);
void launch_gw_reduce(const cgb200_plan* p, const float2* partial, int slices, float2* gW, cudaStream_t st);
int64_t tc_pack_floats(const cgb200_plan* p);
int tc_fwd_level(const cgb200_plan* p, int64_t G);
int64_t gff_pack_floats(const cgb200_plan* p);
int64_t gff_group_elems(const cgb200_plan* p);
int launch_gff_tc(const cgb200_plan* p, int lv, const float2* SG, const float2* W, const float* inv, float* pack, float2* gff,
                  int G, cudaStream_t st);
int launch_fwd_tc(const cgb200_plan* p, int lv, const float2* SF, const float2* W, const float* inv, float* pack, float2* O,
                  float2* O_part, int B, int G, const float2* ff, cudaStream_t st);
void launch_parts_reduce(int kid, const int64_t* cum, int n_deg, int64_t n_total, const int* parts, const float2* partial,
                         int64_t part_stride, float2* out, int B, bool skip_single, cudaStream_t st);
}  // namespace cgb200

// The opaque handle of the C ABI.
struct cgb200_plan {
    int device = 0;
    int num_sms = 148;
    int flags = 0;
    int opt[CGB200_OPT_COUNT];        // kernel selection (cgb200_plan_set_option); CGB200_AUTO = the measured default
    cgb200_plan() { for (int& o : opt) o = CGB200_AUTO; }
    cgb200::PlanDev d{};
    std::vector<int> tF, tO, tFF, cumT;
    std::vector<int64_t> cumF, cumFF, cumO, cumW;
    std::vector<int> cumSF, cumSO;
    std::vector<cgb200::TripleRec> triples;
    std::vector<cgb200::CellRec> cells;
    std::vector<cgb200::CellInfo> cell_info;
    std::vector<cgb200::GwTask> gw_tasks;
    const cgb200::GwTask* d_gw_tasks = nullptr;
    std::vector<cgb200::GfInfo> gf_info;
    const cgb200::GfInfo* d_gf_info = nullptr;
    std::vector<int> cell_begin, triple_begin;
    int max_n = 1;                    // 2*lmax+1
    int64_t cg_len = 0;               // floats in the CG table
    std::vector<cgb200::GenItem> gen_items;
    const cgb200::GenItem* d_gen_items = nullptr;
    size_t gen_band_bytes = 0;        // largest CG band of a triple, padded to 16 bytes
    size_t gen_sample_bytes = 0;      // largest zero-padded operand pair of a triple, per sample
    std::vector<int> gw_begin;        // [n_triples+1] warp-tasks of the fused weight-gradient kernel per triple
    int gw_i = 1;                     // t1 channels per weight-gradient task
    int gw_to = 1;                    // output channels per weight-gradient task
    std::vector<cgb200::GfEntry> gf_entries;
    std::vector<int> gf_begin;        // [lmax+2] entries of fragment l
    const int* d_gf_begin = nullptr;
    // blocks of the cell-staged input-gradient kernel for several degrees of splitting: level s splits the entry
    // list of the most expensive fragment s ways and the others in proportion to their cost
    static constexpr int kGfLevels = 6;               // s = 1, 2, 4, 8, 16, 32
    std::vector<int> gf2_blocks[kGfLevels];           // (fragment, owned tile, part, parts) per block
    const int* d_gf2_blocks[kGfLevels] = {nullptr};
    std::vector<unsigned char> gf_owner;   // warp of every phase-2 unit of the input-gradient kernel, [2 l^2 + u]
    const unsigned char* d_gf_owner = nullptr;
    std::vector<int> gf2_parts[kGfLevels];            // [lmax+1] parts per fragment
    const int* d_gf2_parts[kGfLevels] = {nullptr};
    int gf2_max_parts[kGfLevels] = {0};
    double gf2_longest[kGfLevels] = {0};             // modelled cost of the longest block of a level (units below)
    double gf_total_cost = 0;                         // modelled cost of all blocks of one sample group
    // tensor-core forward (tile edge 2 or 4, full product): per degree the padded GEMM width N' = 2*tau_out rounded
    // up to 16, the offset (in floats) of the degree's packed weights, and the list of row tiles (l, first m index)
    bool tc_ok = false;
    bool tc_gw_ok = false;            // the tensor-core weight gradient's tables exist (tile edge 4 or 5)
    std::vector<int> tc_npad;
    std::vector<int64_t> tc_pack_off;   // [lmax+2]
    // Row tiles of the tensor-core forward, per splitting level: (l, first m index, part, parts) with the longest
    // contraction first.  At level v the degree with the most cells is cut into 2^v parts of its cells and every other
    // degree into as many parts as keep its parts no longer than that; a part writes a partial output that
    // parts_reduce_kernel adds up in part order.
    static constexpr int kTcLevels = 7;
    std::vector<int> tc_tiles[kTcLevels];
    const int* d_tc_tiles[kTcLevels] = {nullptr};
    std::vector<int> tc_parts[kTcLevels];           // [lmax+1] parts per degree
    const int* d_tc_parts[kTcLevels] = {nullptr};
    int tc_max_parts[kTcLevels] = {0};
    int tc_longest[kTcLevels] = {0};                // cells of the longest part
    int64_t tc_total_cells = 0;                     // cells summed over the row tiles of one sample group
    const int* d_tc_npad = nullptr;
    const int64_t* d_tc_pack_off = nullptr;
    // mid-activation gradient as a tensor-core GEMM (tile edge 4, full product): per degree the offset of its packed
    // weights (floats) and of its tiles inside one sample group of the gradient workspace (units of 32 lanes of float2;
    // the tile of a degree's cell k starts at offset + k (2l+1) T^2)
    bool gff_ok = false;     // the mid-gradient GEMM's tables exist (tile edge 4, tensor-core tables)
    bool tiles_ok = false;   // gff_off exists: the mid activation can be kept as tiles (full product, any tile edge)
    std::vector<int64_t> gff_pack_off, gff_off;   // [lmax+2]
    const int64_t* d_gff_pack_off = nullptr;
    const int64_t* d_gff_off = nullptr;
    std::vector<int> tc_gw_tiles;       // tensor-core weight gradient: (l, first cell of a block of four) pairs, longest first
    const int* d_tc_gw_tiles = nullptr;
    // CG table with every band row padded to a multiple of four floats (16-byte aligned rows: the four band rows a row
    // tile of the staged tensor-core forward needs are then one cp.async.bulk), and each cell's offset into it
    const float* d_cg_pad = nullptr;
    std::vector<int> cell_cgpad;
    const int* d_cell_cgpad = nullptr;
    int* d_status = nullptr;          // set to 1 by a kernel whose bounded wait ran out (cgb200_plan_status)
    std::vector<int> fwd_rows;        // (l, m+l) rows of the output, most expensive first (dynamic scheduling order)
    const int* d_fwd_rows = nullptr;
    int max_tau_out = 0;
    std::vector<void*> allocations;   // every cudaMalloc of the plan, freed on destroy

    // cgb200_layer_bwd runs the weight gradient beside the input gradient: a second stream forked from and joined
    // back to the caller's stream with these two events (created on first use; the mutex keeps one call's
    // fork ... join enqueue sequence from interleaving with another thread's on the same plan)
    mutable cudaStream_t side_stream = nullptr;
    mutable cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    mutable std::mutex side_mutex;
};

namespace cgb200 {
inline uint32_t wait_polls(const cgb200_plan* p) {
    const int v = p->opt[CGB200_OPT_WAIT_POLLS];
    return v > 0 ? (uint32_t)v : kDefaultWaitPolls;
}
}  // namespace cgb200

#ifdef __CUDACC__
namespace cgb200 {

__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
// acc += a * b
__device__ __forceinline__ void cfma(float2& acc, float2 a, float2 b) {
    acc.x = fmaf(a.x, b.x, acc.x);
    acc.x = fmaf(-a.y, b.y, acc.x);
    acc.y = fmaf(a.x, b.y, acc.y);
    acc.y = fmaf(a.y, b.x, acc.y);
}
// acc += conj(a) * b
__device__ __forceinline__ void cfma_conj(float2& acc, float2 a, float2 b) {
    acc.x = fmaf(a.x, b.x, acc.x);
    acc.x = fmaf(a.y, b.y, acc.x);
    acc.y = fmaf(a.x, b.y, acc.y);
    acc.y = fmaf(-a.y, b.x, acc.y);
}

// Register-tiled generator of CG-product values for one sample and one m.  Full product (DW == false):
//     v[i*T + j] = sum_{m2} C[m][m2] * F1[i][m - m2] * F2[j][m2],     i < T, j < T
// depthwise product (DW == true):
//     v[i]       = sum_{m2} C[m][m2] * F1[i][m - m2] * F2[i][m2],     i < T
// (CGNet/cudaCG/cudaCG_sparse.cu:162-174 computes a single (i, j) per thread).  Per m2 step a thread of the full
// product loads 2T+1 values for 4*T*T fused multiply-adds, which keeps the loop arithmetic-bound for T >= 3.
//   Crow   the band row of this m, indexed by m2 + l2
//   F1     rows of the first operand, row stride s1 (>= 2*l1+1), element [i*s1 + (m1 + l1)]; rows beyond the
//          fragment's channel count must be readable (callers stage zero-padded tiles or over-allocate) and their
//          results are masked by the caller through tile_valid()
//   F2     likewise for the second operand with row stride s2
//   es     distance between consecutive elements of a row (1 for a plain row; the padded batch size when the
//          operands are stored sample-fastest and every lane of the warp reads its own sample)
template <int T, bool DW>
struct TileShape {
    static constexpr int NV = DW ? T : T * T;
};

template <int T, bool DW>
__device__ __forceinline__ void gen_tile(float2 (&v)[TileShape<T, DW>::NV], const float* __restrict__ Crow,
                                         const float2* __restrict__ F1, int s1, const float2* __restrict__ F2, int s2,
                                         int m, int l1, int l2, int64_t es = 1) {
    constexpr int NV = TileShape<T, DW>::NV;
    const int lo = max(-l2, m - l1), hi = min(l2, m + l1);
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = make_float2(0.f, 0.f);
    for (int m2 = lo; m2 <= hi; ++m2) {
        const float c = Crow[m2 + l2];
        float2 b[T];
#pragma unroll
        for (int j = 0; j < T; ++j) b[j] = F2[(int64_t)(j * s2 + m2 + l2) * es];
#pragma unroll
        for (int i = 0; i < T; ++i) {
            float2 a = F1[(int64_t)(i * s1 + (m - m2) + l1) * es];
            a.x *= c;
            a.y *= c;
            if (DW) {
                cfma(v[i], a, b[i]);
            } else {
#pragma unroll
                for (int j = 0; j < T; ++j) cfma(v[i * T + j], a, b[j]);
            }
        }
    }
}

// The same generator for operands in slab layout (see PlanDev): S1 / S2 point at this lane's element (m = -l, channel
// 0) of the t1 tile / t2 tile, so the T channels of a tile at one m are 32 float2 apart and consecutive m are T*32
// apart: every inner-loop offset is a compile-time constant.  Works for global and for shared-memory slabs.
template <int T, bool DW, bool PIPE = false>
__device__ __forceinline__ void gen_slab(float2 (&v)[TileShape<T, DW>::NV], const float* __restrict__ Crow,
                                         const float2* __restrict__ S1, const float2* __restrict__ S2, int m, int l1,
                                         int l2) {
    constexpr int NV = TileShape<T, DW>::NV;
    const int lo = max(-l2, m - l1), hi = min(l2, m + l1);
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = make_float2(0.f, 0.f);
    const float2* p2 = S2 + (lo + l2) * (T * 32);
    const float2* p1 = S1 + (m - lo + l1) * (T * 32);
    const float* pc = Crow + lo + l2;
    if constexpr (PIPE) {
        // Software pipeline for operands that come from global memory through L1: the loads of band step k+1 are in
        // flight while step k's FMAs run (the last step fetches its own operands again, which keeps the loop free of
        // a peeled tail and every address inside the band).  Measured: 7 % faster statistics kernel, but slower
        // where the operands sit in shared memory (more registers, nothing to hide), so it is opt-in.
        if (hi < lo) return;
        float c = *pc;
        float2 a[T], b[T];
#pragma unroll
        for (int j = 0; j < T; ++j) b[j] = p2[j * 32];
#pragma unroll
        for (int i = 0; i < T; ++i) a[i] = p1[i * 32];
        for (int k = hi - lo; k >= 0; --k) {
            const int adv = k > 0 ? 1 : 0;
            pc += adv;
            p2 += adv * (T * 32);
            p1 -= adv * (T * 32);
            const float cn = *pc;
            float2 an[T], bn[T];
#pragma unroll
            for (int j = 0; j < T; ++j) bn[j] = p2[j * 32];
#pragma unroll
            for (int i = 0; i < T; ++i) an[i] = p1[i * 32];
#pragma unroll
            for (int i = 0; i < T; ++i) {
                const float2 ac = make_float2(a[i].x * c, a[i].y * c);
                if (DW) {
                    cfma(v[i], ac, b[i]);
                } else {
#pragma unroll
                    for (int j = 0; j < T; ++j) cfma(v[i * T + j], ac, b[j]);
                }
            }
            c = cn;
#pragma unroll
            for (int j = 0; j < T; ++j) b[j] = bn[j];
#pragma unroll
            for (int i = 0; i < T; ++i) a[i] = an[i];
        }
    } else {
        for (int k = hi - lo; k >= 0; --k) {
            const float c = *pc++;
            float2 b[T];
#pragma unroll
            for (int j = 0; j < T; ++j) b[j] = p2[j * 32];
#pragma unroll
            for (int i = 0; i < T; ++i) {
                float2 a = p1[i * 32];
                a.x *= c;
                a.y *= c;
                if (DW) {
                    cfma(v[i], a, b[i]);
                } else {
#pragma unroll
                    for (int j = 0; j < T; ++j) cfma(v[i * T + j], a, b[j]);
                }
            }
            p2 += T * 32;
            p1 -= T * 32;
        }
    }
}

// The generator restricted to the rows I0 .. I0+IN of the tile (full product only): v[i*T + j] for i < IN is the tile's
// entry (I0 + i, j).  Operand loads software-pipelined as in gen_slab<.., true>.
template <int T, int I0, int IN>
__device__ __forceinline__ void gen_slab_rows(float2 (&v)[IN * T], const float* __restrict__ Crow, const float2* __restrict__ S1,
                                              const float2* __restrict__ S2, int m, int l1, int l2) {
    const int lo = max(-l2, m - l1), hi = min(l2, m + l1);
#pragma unroll
    for (int i = 0; i < IN * T; ++i) v[i] = make_float2(0.f, 0.f);
    if (hi < lo) return;
    const float2* p2 = S2 + (lo + l2) * (T * 32);
    const float2* p1 = S1 + (m - lo + l1) * (T * 32) + I0 * 32;
    const float* pc = Crow + lo + l2;
    float c = *pc;
    float2 a[IN], b[T];
#pragma unroll
    for (int j = 0; j < T; ++j) b[j] = p2[j * 32];
#pragma unroll
    for (int i = 0; i < IN; ++i) a[i] = p1[i * 32];
    for (int k = hi - lo; k >= 0; --k) {
        const int adv = k > 0 ? 1 : 0;   // the last step fetches its own operands again: no peeled tail, no stray address
        pc += adv;
        p2 += adv * (T * 32);
        p1 -= adv * (T * 32);
        const float cn = *pc;
        float2 an[IN], bn[T];
#pragma unroll
        for (int j = 0; j < T; ++j) bn[j] = p2[j * 32];
#pragma unroll
        for (int i = 0; i < IN; ++i) an[i] = p1[i * 32];
#pragma unroll
        for (int i = 0; i < IN; ++i) {
            const float2 ac = make_float2(a[i].x * c, a[i].y * c);
#pragma unroll
            for (int j = 0; j < T; ++j) cfma(v[i * T + j], ac, b[j]);
        }
        c = cn;
#pragma unroll
        for (int j = 0; j < T; ++j) b[j] = bn[j];
#pragma unroll
        for (int i = 0; i < IN; ++i) a[i] = an[i];
    }
}

// Mid channel (relative to the triple's first) of tile entry idx, and whether the entry exists.
template <int T, bool DW>
__device__ __forceinline__ int tile_channel(int idx, int t1_0, int t2_0, int tau2) {
    return DW ? (t1_0 + idx) : ((t1_0 + idx / T) * tau2 + t2_0 + idx % T);
}
template <int T, bool DW>
__device__ __forceinline__ bool tile_valid(int idx, int t1_0, int t2_0, int tau1, int tau2) {
    return DW ? (t1_0 + idx < tau1) : ((t1_0 + idx / T < tau1) && (t2_0 + idx % T < tau2));
}

// Largest k with cum[k] <= e, for a non-decreasing table cum[0..n] (cum[0] == 0, e < cum[n]).
__device__ __forceinline__ int find_degree(const int64_t* __restrict__ cum, int n, int64_t e) {
    int lo = 0, hi = n;   // invariant: cum[lo] <= e < cum[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cum[mid] <= e) lo = mid; else hi = mid;
    }
    return lo;
}

// ---- pieces of the fused input-gradient kernels (CUDA-core and tensor-core variant) ----------------------------------
// Work split inside a block.  A phase ends at a barrier, so it lasts as long as its busiest warp:
//   phase 1  unit = (m, half of the tile's NH entries), all of about equal cost, dealt round-robin;
//   phase 2  unit = a row of the owned fragment (or, optionally, its first ceil(T/2) / last floor(T/2) owned channels);
//            a unit's cost follows the row's band length, and the plan holds a longest-processing-time assignment of
//            every owned degree's units to the 16 warps (table `owner`, index 2 l^2 + u for unit u of degree l).
template <int T, bool DW>
struct GfShape {
    static constexpr int NH = DW ? T : T * T;
    static constexpr int NHP = (NH + 1) & ~1;                   // row pitch of the staged weights: 16-byte rows
    static constexpr int KA = NH >= 4 ? ((NH / 2) & ~1) : 0;    // entries of phase 1's first half (even), 0: no split
    static constexpr int AH = (T + 1) / 2;                      // owned channels of phase 2's heavy unit
    static constexpr int AL = T - AH;                           // ... of its light unit (0 for T = 1: no split)
};

// phase 2 unit: owned channels A0 .. A0+AN of row r gather their band from the H tiles of the chunk
template <int T, bool DW, bool FIRST, int A0, int AN>
__device__ __forceinline__ void gf_row_unit(const float2* __restrict__ H, const float2* __restrict__ fo,
                                            const float* __restrict__ band, float2* __restrict__ acc, int r, int lt, int nt,
                                            int l, int lo_, int l2, int n2, int mc0, int mcn, int lane) {
    constexpr int NH = DW ? T : T * T;
    float2 x[AN];
#pragma unroll
    for (int a = 0; a < AN; ++a) x[a] = make_float2(0.f, 0.f);
    const int mt = r - lt;
    // m = m_t + u with u = m of the other operand's element, |u| <= lo_, m inside [-l, l] and inside the chunk
    const int mlo = max(max(-l, mc0 - l), mt - lo_), mhi = min(min(l, mc0 + mcn - 1 - l), mt + lo_);
    for (int m = mlo; m <= mhi; ++m) {
        const int u = m - mt;
        const float cg = band[(m + l) * n2 + (FIRST ? u : mt) + l2];   // band entry [m + l][m2 + l2]
        const float2* ph = H + (size_t)(m + l - mc0) * NH * 32 + lane;
        const float2* pf = fo + (size_t)(u + lo_) * T * 32 + lane;
        if constexpr (DW) {
#pragma unroll
            for (int a = 0; a < AN; ++a) {
                const float2 f = pf[(A0 + a) * 32];
                cfma_conj(x[a], make_float2(f.x * cg, f.y * cg), ph[(A0 + a) * 32]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < T; ++c) {
                float2 f = pf[c * 32];
                f.x *= cg;
                f.y *= cg;
#pragma unroll
                for (int a = 0; a < AN; ++a) cfma_conj(x[a], f, ph[(FIRST ? (A0 + a) * T + c : c * T + A0 + a) * 32]);
            }
        }
    }
#pragma unroll
    for (int a = 0; a < AN; ++a) {
        float2* pa = acc + ((size_t)(A0 + a) * nt + r) * 32 + lane;
        float2 cur = *pa;
        cur.x += x[a].x;
        cur.y += x[a].y;
        *pa = cur;
    }
}

// One phase-2 unit of a block.  Without the split a unit is a whole row (all T owned channels); with it, units
// 0 .. nt-1 carry the first ceil(T/2) owned channels of their row and units nt .. 2 nt-1 the rest.  Measured on B200 the
// whole-row units win at every shape tried (tile edges 3, 4, 5; 3 to 32 channels) by 2-8 %; rows in groups of two or
// three, which load a gFF tile element once for several rows, were 10-80 % slower (fewer, longer units on 16 warps).
template <int T, bool DW, bool SPLIT>
__device__ __forceinline__ void gf_phase2_unit(int u, bool first, const float2* __restrict__ H, const float2* __restrict__ fo,
                                               const float* __restrict__ band, float2* __restrict__ acc, int lt, int nt, int l,
                                               int lo_, int l2, int n2, int mc0, int mcn, int lane) {
    using S = GfShape<T, DW>;
    constexpr bool kSplit = SPLIT && S::AL > 0;
    constexpr int AH = kSplit ? S::AH : T;
    const bool heavy = u < nt;
    const int r = heavy ? u : u - nt;
    if (heavy) {
        if (first) gf_row_unit<T, DW, true, 0, AH>(H, fo, band, acc, r, lt, nt, l, lo_, l2, n2, mc0, mcn, lane);
        else gf_row_unit<T, DW, false, 0, AH>(H, fo, band, acc, r, lt, nt, l, lo_, l2, n2, mc0, mcn, lane);
    } else if constexpr (kSplit) {
        if (first) gf_row_unit<T, DW, true, S::AH, S::AL>(H, fo, band, acc, r, lt, nt, l, lo_, l2, n2, mc0, mcn, lane);
        else gf_row_unit<T, DW, false, S::AH, S::AL>(H, fo, band, acc, r, lt, nt, l, lo_, l2, n2, mc0, mcn, lane);
    }
}
// number of phase-2 units of a block that owns a fragment with nt rows
template <int T, bool DW, bool SPLIT>
__device__ __forceinline__ int gf_phase2_units(int nt) {
    return ((SPLIT && GfShape<T, DW>::AL > 0) ? 2 : 1) * nt;
}

}  // namespace cgb200
#endif
