// The experts' products of many rows on the fifth-generation tensor cores.
//
// The rows of a step, sorted by expert with every expert's rows starting on a tile boundary (moe_sort_kernel in
// moe.cu), are gathered into one matrix; an output tile of 128 sorted rows belongs to one expert, which a table
// names.  The experts' matrices lie stacked and stored (out, in): for the tensor cores that is the K-major second
// operand, as the keys of attention are, so a TMA box of BN weight rows x 64 elements of K lands as the operand tile
// it is, and a tile's expert only moves the box's row coordinate.
//   gated   C[rows][h] = silu(x . Wg[e][h]) * (x . Wu[e][h]): the box of a tile's gate rows and the box of its up rows
//           form one operand of BN = 2 x BH rows; the accumulator's first BH columns are the gates, the others the ups.
//   plain   C[rows][c] = x . Wd[e][c].
// Roles, hand-offs, bounded waits and the double-buffered accumulator are those of gemm_tc.cu; tiles whose table entry
// is negative (beyond the last expert's rows) are skipped by every role alike.
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int NTH = 192;
constexpr int A_BYTES = BM * BK * 2;

struct MoeTcParams {
    bf16* out; int ldo;
    int N;                  // output columns: hidden elements (gated) or the model's width
    int K;
    int rows_per_expert;    // rows of the stacked weight matrix that one expert holds (2 x hidden, or width)
    int up_offset;          // gated: the expert's up rows start this many rows after its gate rows
    int tiles_m, tiles_n;
    const int* tile_expert;
    int* fault;
    int act;                // not gated: -1 none, else the activation of the output (0 relu^2, 1 gelu (tanh), 2 silu)
};

__device__ __forceinline__ float tile_act(float x, int kind) {
    if (kind == 0) { const float r = fmaxf(x, 0.f); return r * r; }
    if (kind == 1) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    return x / (1.f + __expf(-x));
}

template <int BN, int STAGES, bool GATED>
__global__ void __launch_bounds__(NTH, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const MoeTcParams p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BH = GATED ? BN / 2 : BN;                // output columns of a tile
    constexpr unsigned TMEM_COLS = BN > 128 ? 512 : 256;
    constexpr unsigned IDESC = instr_desc(BM, BN, false);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kt_count = p.K / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_map(&map_a);
        prefetch_map(&map_b);
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;
    pdl_wait();                                           // the rows and the table are the output of kernels before

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x) {
                const int tm = tile % p.tiles_m, e = p.tile_expert[tm];
                if (e < 0) continue;
                const int m0 = tm * BM, n0 = (tile / p.tiles_m) * BH;
                const int w_row = e * p.rows_per_expert + n0;
                bool ok = true;
                for (int kt = 0; kt < kt_count; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort, p.fault, 7)) { ok = false; break; }
                    unsigned char* a = tiles + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a, &map_a, kt * BK, m0, &full[s]);
                    tma_load_2d(a + A_BYTES, &map_b, kt * BK, w_row, &full[s]);
                    if (GATED) tma_load_2d(a + A_BYTES + BH * BK * 2, &map_b, kt * BK, w_row + p.up_offset, &full[s]);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, acc_it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x) {
                if (p.tile_expert[tile % p.tiles_m] < 0) continue;
                const int b = acc_it & 1;
                if (!mbar_wait(&acc_empty[b], ((acc_it >> 1) & 1) ^ 1, abort, p.fault, 7)) break;
                fence_after();
                const unsigned d = tmem_base + b * BN;
                bool ok = true;
                for (int kt = 0; kt < kt_count; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1, abort, p.fault, 7)) { ok = false; break; }
                    fence_after();
                    const unsigned a = smem_u32(tiles + s * STAGE_BYTES), w = a + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // both operands K-major: 16 elements of K further = 32 bytes inside the swizzled 128-byte row
                        const unsigned long long da = smem_desc(a + kk * 32, 16, 1024);
                        const unsigned long long db = smem_desc(w + kk * 32, 16, 1024);
                        umma(d, da, db, IDESC, (kt | kk) != 0);
                    }
                    umma_commit(&empty[s]);
                }
                if (!ok) break;
                umma_commit(&acc_full[b]);
                ++acc_it;
            }
        }
    } else {
        const int quarter = warp & 3;
        int acc_it = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x) {
            const int tm = tile % p.tiles_m;
            if (p.tile_expert[tm] < 0) continue;
            const int b = acc_it & 1;
            const int m0 = tm * BM, n0 = (tile / p.tiles_m) * BH;
            if (!mbar_wait(&acc_full[b], (acc_it >> 1) & 1, abort, p.fault, 7)) break;
            fence_after();
            const size_t row = (size_t)m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + b * BN;
#pragma unroll 1
            for (int c = 0; c < BH / 32; ++c) {
                float g[32];
                tmem_ld32(taddr + c * 32, g);
                if (GATED) {
                    float u[32];
                    tmem_ld32(taddr + BH + c * 32, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) g[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
                } else if (p.act >= 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) g[i] = tile_act(g[i], p.act);
                }
                bf16* o = p.out + row * p.ldo + n0 + c * 32;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (n0 + c * 32 + q * 8 < p.N) store8(o + q * 8, g + q * 8);
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
            ++acc_it;
        }
    }

    if (*abort) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tmem_base, TMEM_COLS);
    }
}

// xs[place] = x[pair / top] for every place of the sorted order that a (token, choice) pair takes; 16-byte vectors.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ sorted_pair, int top, bf16* __restrict__ xs,
                  int d) {
    pdl_launch_dependents();
    const int place = blockIdx.x;
    pdl_wait();
    const int pair = sorted_pair[place];
    if (pair < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / top) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)place * d);
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

template <int BN, int STAGES, bool GATED>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, MoeTcParams p, cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + BN * BK * 2) + 1024;
    static bool configured = false;
    auto kernel = moe_tc_kernel<BN, STAGES, GATED>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return tis_check_launch("moe_tc (shared memory)");
        configured = true;
    }
    p.tiles_n = (p.N + (GATED ? BN / 2 : BN) - 1) / (GATED ? BN / 2 : BN);
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    tis_launch(kernel, dim3(grid), dim3(NTH), (size_t)smem, stream, ma, mb, p);
    return tis_check_launch("moe_tc");
}

}  // namespace

// defined in moe.cu: the sort with tiles of `tile_rows` rows, and the weighted sum of the chosen experts' outputs
int tis_moe_sort_launch(const int* chosen, int pairs, int E, int tile_rows, int* sorted_pair, int max_rows, int* pair_place,
                        int* tile_expert, int max_tiles, cudaStream_t stream);
int tis_moe_combine_launch(const void* y, int ldy, const int* pair_place, const float* weights, const void* shared, int lds,
                           const float* shared_gate, void* out, int n, int d, int top, cudaStream_t stream);

// Tiles of 128 sorted rows that `pairs` (token, choice) pairs over E experts can need at most.
TIS_API int tis_moe_tc_tiles(int pairs, int E) { return (pairs + BM - 1) / BM + E; }

// The experts' products for many rows in bfloat16 on the tcgen05 tensor cores.  x (n, d) with row stride ldx; w_gu
// (E, 2, F, d), or (E, F, d) with act >= 0 (units without a gate, the activation on the first product); w_down (E, d, F); scratch for T = tis_moe_tc_tiles(n * top, E) tiles: sorted_pair T * 128, pair_place
// n * top, tile_expert T, xs (T * 128, d), hidden (T * 128, F), y (T * 128, d).  d and F multiples of 64.
TIS_API int tis_moe_grouped_tc(const void* x, int ldx, const int* chosen, const float* weights, const void* w_gu,
                               const void* w_down, const void* shared, int lds, const float* shared_gate, void* out,
                               int* sorted_pair, int* pair_place, int* tile_expert, void* xs, void* hidden, void* y, int n,
                               int d, int top, int E, int F, int act, int* fault, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || F <= 0 || d % BK || F % BK || ldx % 8 || lds % 2 || E <= 0 || E > 4096 || top <= 0 ||
        ((uintptr_t)x | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)xs | (uintptr_t)hidden | (uintptr_t)y) % 16 ||
        ((uintptr_t)shared | (uintptr_t)out) % 4) {
        tis_set_error("moe_grouped_tc: width %d and hidden %d must be multiples of %d, operands aligned (%d experts, top %d)",
                      d, F, BK, E, top);
        return TIS_BAD_SIZE;
    }
    const int pairs = n * top, tiles_m = tis_moe_tc_tiles(pairs, E), rows = tiles_m * BM;
    int st = tis_moe_sort_launch(chosen, pairs, E, BM, sorted_pair, rows, pair_place, tile_expert, tiles_m, stream);
    if (st != TIS_OK) return st;
    tis_launch(moe_gather_kernel, dim3(rows), dim3(d / 8 < 256 ? (d / 8 + 31) / 32 * 32 : 256), 0, stream, (const bf16*)x, ldx,
               (const int*)sorted_pair, top, (bf16*)xs, d);
    st = tis_check_launch("moe_gather");
    if (st != TIS_OK) return st;
    CUtensorMap ma, mb;
    MoeTcParams p;
    p.fault = fault;
    p.tile_expert = tile_expert;
    p.tiles_m = tiles_m;
    p.tiles_n = 0;
    // gate and up with the gating: K = d, the stacked matrix has E * 2F rows of d elements
    p.out = static_cast<bf16*>(hidden); p.ldo = F; p.N = F; p.K = d; p.rows_per_expert = 2 * F; p.up_offset = F;
    p.act = -1;
    if (act >= 0) {
        // units without a gate: one matrix of F rows an expert, the activation in the epilogue
        p.rows_per_expert = F; p.up_offset = 0; p.act = act;
        if (F >= 256) {
            if (!tensor_map(xs, d, rows, d, BM, true, &ma) || !tensor_map(w_gu, d, (long long)E * F, d, 256, true, &mb))
                return TIS_CUDA_ERROR;
            st = launch<256, 4, false>(ma, mb, p, stream);
        } else {
            if (!tensor_map(xs, d, rows, d, BM, true, &ma) || !tensor_map(w_gu, d, (long long)E * F, d, 128, true, &mb))
                return TIS_CUDA_ERROR;
            st = launch<128, 6, false>(ma, mb, p, stream);
        }
    } else if (F >= 128) {
        if (!tensor_map(xs, d, rows, d, BM, true, &ma) || !tensor_map(w_gu, d, (long long)E * 2 * F, d, 128, true, &mb))
            return TIS_CUDA_ERROR;
        st = launch<256, 4, true>(ma, mb, p, stream);
    } else {
        if (!tensor_map(xs, d, rows, d, BM, true, &ma) || !tensor_map(w_gu, d, (long long)E * 2 * F, d, 64, true, &mb))
            return TIS_CUDA_ERROR;
        st = launch<128, 6, true>(ma, mb, p, stream);
    }
    if (st != TIS_OK) return st;
    // down: K = F, the stacked matrix has E * d rows of F elements
    p.out = static_cast<bf16*>(y); p.ldo = d; p.N = d; p.K = F; p.rows_per_expert = d; p.up_offset = 0; p.act = -1;
    if (d >= 256) {
        if (!tensor_map(hidden, F, rows, F, BM, true, &ma) || !tensor_map(w_down, F, (long long)E * d, F, 256, true, &mb))
            return TIS_CUDA_ERROR;
        st = launch<256, 4, false>(ma, mb, p, stream);
    } else {
        if (!tensor_map(hidden, F, rows, F, BM, true, &ma) || !tensor_map(w_down, F, (long long)E * d, F, 128, true, &mb))
            return TIS_CUDA_ERROR;
        st = launch<128, 6, false>(ma, mb, p, stream);
    }
    if (st != TIS_OK) return st;
    return tis_moe_combine_launch(y, d, pair_place, weights, shared, lds, shared_gate, out, n, d, top, stream);
}
