// A mixture of small gated feed-forward units: the router, and the experts' products for the experts that each row
// chose.  The experts' matrices are stacked and stored (out, in), so that an output element is one dot product over
// contiguous weights; a kernel finds an expert's matrix from the row's choice on the device, nothing is sorted or
// gathered.  Sums are 32-bit; T is the storage type of activations and weights.
#include "common.cuh"

namespace {

constexpr int MOE_THREADS = 128;

// ND dot products at once, out[j] = sum_i w[j][i] * x[j][i] over a warp: the loads of all of them are in flight together,
// which is what a kernel that streams weights once lives on.
//
// The x of a vector path lie in shared memory as fill_f32 leaves them: for vectors of four elements in their own order;
// for vectors of eight as two planes, elements 0..3 of every group of eight in the first half of the array and elements
// 4..7 in the second, so that the 16-byte reads of neighbouring lanes are neighbours and meet no bank twice.
template <typename T, int ND>
__device__ __forceinline__ void warp_dots(const T* const (&w)[ND], const float* const (&x)[ND], int d, int lane, bool vec,
                                          float (&out)[ND]) {
    constexpr int N = Vec16<T>::N;
    float acc[ND];
#pragma unroll
    for (int j = 0; j < ND; ++j) acc[j] = 0.f;
    if (vec) {
#pragma unroll(ND * N >= 32 ? 2 : 4)
        for (int i = lane * N; i < d; i += 32 * N) {
            float v[ND][N];
#pragma unroll
            for (int j = 0; j < ND; ++j) Vec16<T>::load(w[j] + i, v[j]);
#pragma unroll
            for (int j = 0; j < ND; ++j) {
                float xv[N];
                if (N == 8) {
                    const float4 a = *reinterpret_cast<const float4*>(x[j] + (i >> 1));
                    const float4 b = *reinterpret_cast<const float4*>(x[j] + (d >> 1) + (i >> 1));
                    xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
                    xv[N - 4] = b.x; xv[N - 3] = b.y; xv[N - 2] = b.z; xv[N - 1] = b.w;
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(x[j] + i);
                    xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
                }
#pragma unroll
                for (int e = 0; e < N; ++e) acc[j] = fmaf(v[j][e], xv[e], acc[j]);
            }
        }
    } else {
        for (int i = lane; i < d; i += 32)
#pragma unroll
            for (int j = 0; j < ND; ++j) acc[j] = fmaf(to_f32(w[j][i]), x[j][i], acc[j]);
    }
#pragma unroll
    for (int j = 0; j < ND; ++j) out[j] = warp_sum(acc[j]);
}

// dst = float(src[0 .. count)) by all threads of the CTA.  `vec`: 16-byte loads, and for vectors of eight elements (PLANES)
// the two planes that warp_dots reads; else element by element in order.
template <typename T, bool PLANES>
__device__ __forceinline__ void fill_f32(float* dst, const T* __restrict__ src, int count, bool vec) {
    constexpr int N = Vec16<T>::N;
    if (vec) {
        float v[N];
        for (int i = threadIdx.x * N; i < count; i += blockDim.x * N) {
            Vec16<T>::load(src + i, v);
            if (PLANES && N == 8) {
                *reinterpret_cast<float4*>(dst + (i >> 1)) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(dst + (count >> 1) + (i >> 1)) = make_float4(v[N - 4], v[N - 3], v[N - 2], v[N - 1]);
            } else {
#pragma unroll
                for (int e = 0; e < N; ++e) dst[i + e] = v[e];
            }
        }
    } else {
        for (int i = threadIdx.x; i < count; i += blockDim.x) dst[i] = to_f32(src[i]);
    }
}

// ------------------------------------------------------------------------------------------------------------
// The router, a CTA a row:  s = sigmoid(W x) over E experts (W float32 (E, d));  pick = s + correction;  with
// groups > 0 the experts form that many groups of E / groups neighbours, a group's strength is the sum of its two
// largest picks, and only the experts of the `keep` strongest groups stay in the race;  the `top` largest picks
// win (the lower index on a tie);  weights: their s over the sum of those (+ weight_eps).  Also sigmoid(w_sg . x)
// if w_sg is given.  score_kind 1: the logits themselves are the picks (correction added if given) and the weights are
// the softmax over the chosen experts' logits only.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(2 * MOE_THREADS)
moe_route_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ wr, const float* __restrict__ corr,
                 const float* __restrict__ w_sg, int d, int E, int groups, int keep, int top, float weight_eps,
                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate, int score_kind) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                  // [d]
    float* sc = xs + d;                // [E]  sigmoid scores
    float* pick = sc + E;              // [E]  choosing scores; -inf once out of the race
    float* strength = pick + E;        // [groups]
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    fill_f32<T, false>(xs, x + (size_t)r * ldx, d, d % Vec16<T>::N == 0 && (uintptr_t)(x + (size_t)r * ldx) % 16 == 0);
    __syncthreads();
    const bool vec = d % 4 == 0 && ((uintptr_t)wr | (uintptr_t)w_sg) % 16 == 0;
    const int n_dots = E + (w_sg != nullptr ? 1 : 0);
    for (int e0 = 2 * warp; e0 < n_dots; e0 += 2 * nw) {          // a warp takes two experts at a time
        const int e1 = min(e0 + 1, n_dots - 1);
        const float* const w2[2] = {e0 < E ? wr + (size_t)e0 * d : w_sg, e1 < E ? wr + (size_t)e1 * d : w_sg};
        const float* const x2[2] = {xs, xs};
        float z[2];
        warp_dots<float, 2>(w2, x2, d, lane, vec, z);
        if (lane == 0) {
            for (int j = 0; j < (e1 != e0 ? 2 : 1); ++j) {
                const int e = j == 0 ? e0 : e1;
                const float s = (score_kind == 1 && e < E) ? z[j] : 1.f / (1.f + expf(-z[j]));
                if (e < E) { sc[e] = s; pick[e] = s + (corr != nullptr ? corr[e] : 0.f); }
                else shared_gate[r] = s;
            }
        }
    }
    __syncthreads();
    if (tid != 0) return;
    if (groups > 0) {
        const int per = E / groups;
        for (int g = 0; g < groups; ++g) {
            float a = -INFINITY, b = -INFINITY;            // the two largest picks of the group
            for (int i = 0; i < per; ++i) {
                const float v = pick[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            strength[g] = per > 1 ? a + b : a;
        }
        // the `keep` strongest groups stay; a kept group's strength is set to +inf as its mark
        for (int k = 0; k < keep; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int g = 0; g < groups; ++g)
                if (strength[g] != INFINITY && (best < 0 || strength[g] > bv)) { best = g; bv = strength[g]; }
            if (best >= 0) strength[best] = INFINITY;      // kept
        }
        for (int g = 0; g < groups; ++g)
            if (strength[g] != INFINITY)
                for (int i = 0; i < per; ++i) pick[g * per + i] = -INFINITY;
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (pick[e] > bv) { best = e; bv = pick[e]; }
        if (best < 0) best = 0;                            // cannot happen: top never exceeds the experts in the race
        pick[best] = -INFINITY;
        chosen[(size_t)r * top + k] = best;
        weights[(size_t)r * top + k] = sc[best];
        total += sc[best];
    }
    if (score_kind == 1) {                                 // softmax over the chosen logits
        float big = -INFINITY;
        for (int k = 0; k < top; ++k) big = fmaxf(big, weights[(size_t)r * top + k]);
        total = 0.f;
        for (int k = 0; k < top; ++k) {
            const float e = expf(weights[(size_t)r * top + k] - big);
            weights[(size_t)r * top + k] = e;
            total += e;
        }
        for (int k = 0; k < top; ++k) weights[(size_t)r * top + k] /= total;
        return;
    }
    const float inv = 1.f / (total + weight_eps);
    for (int k = 0; k < top; ++k) weights[(size_t)r * top + k] *= inv;
}

// ------------------------------------------------------------------------------------------------------------
// hidden[r * top + k][j] = silu(Wg[e][j] . x[r]) * (Wu[e][j] . x[r]),  e = chosen[r][k];  w_gu (E, 2, F, d).
// act >= 0: units without a gate, hidden = act(Wu[e][j] . x[r]) with w_gu (E, F, d) and act 0 relu^2, 1 gelu (tanh), 2 silu.
// A CTA per (row and choice, block of COLS hidden columns); a warp a column at a time.
// ------------------------------------------------------------------------------------------------------------
constexpr int MOE_COLS = 16;

__device__ __forceinline__ float unit_act(float x, int kind) {
    if (kind == 0) { const float r = fmaxf(x, 0.f); return r * r; }
    if (kind == 1) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    return x / (1.f + expf(-x));
}

template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ chosen, const T* __restrict__ w_gu,
                   T* __restrict__ hidden, int d, int top, int E, int F, int act) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int pair = blockIdx.x, r = pair / top;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    const int e = chosen[pair];
    if (e < 0 || e >= E) return;
    const bool vec = d % Vec16<T>::N == 0 && ((uintptr_t)w_gu | (uintptr_t)(x + (size_t)r * ldx)) % 16 == 0;
    fill_f32<T, true>(smem, x + (size_t)r * ldx, d, vec);
    __syncthreads();
    const T* wg = w_gu + (size_t)e * (act >= 0 ? 1 : 2) * F * d;
    const T* wu = wg + (size_t)F * d;
    const int j_end = min(F, (int)(blockIdx.y + 1) * MOE_COLS);
    if (act >= 0) {                                        // no gate: two columns are two dot products
        for (int j = blockIdx.y * MOE_COLS + 2 * warp; j < j_end; j += 2 * nw) {
            const int j1 = min(j + 1, j_end - 1);
            const T* const w[2] = {wg + (size_t)j * d, wg + (size_t)j1 * d};
            const float* const x2[2] = {smem, smem};
            float r[2];
            warp_dots<T, 2>(w, x2, d, lane, vec, r);
            if (lane == 0) {
                hidden[(size_t)pair * F + j] = from_f32<T>(unit_act(r[0], act));
                if (j1 != j) hidden[(size_t)pair * F + j1] = from_f32<T>(unit_act(r[1], act));
            }
        }
        return;
    }
    // a warp takes two columns at a time: their gate and up rows are four dot products in flight
    for (int j = blockIdx.y * MOE_COLS + 2 * warp; j < j_end; j += 2 * nw) {
        const int j1 = min(j + 1, j_end - 1);
        const T* const w[4] = {wg + (size_t)j * d, wu + (size_t)j * d, wg + (size_t)j1 * d, wu + (size_t)j1 * d};
        const float* const x4[4] = {smem, smem, smem, smem};
        float r[4];
        warp_dots<T, 4>(w, x4, d, lane, vec, r);
        if (lane == 0) {
            hidden[(size_t)pair * F + j] = from_f32<T>(r[0] / (1.f + expf(-r[0])) * r[1]);
            if (j1 != j) hidden[(size_t)pair * F + j1] = from_f32<T>(r[2] / (1.f + expf(-r[2])) * r[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// out[r][c] = sum_k weights[r][k] * (Wd[e_k][c] . hidden[r * top + k])  (+ shared_gate[r] * shared[r][c]);
// w_down (E, d, F).  A CTA per (row, block of COLS output columns).
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(const T* __restrict__ hidden, const int* __restrict__ chosen, const float* __restrict__ weights,
                const T* __restrict__ w_down, const T* __restrict__ shared, int lds,
                const float* __restrict__ shared_gate, T* __restrict__ out, int d, int top, int E, int F) {
    extern __shared__ __align__(16) float smem[];                // [top][F]
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    const bool vec = F % Vec16<T>::N == 0 && ((uintptr_t)w_down | (uintptr_t)hidden) % 16 == 0;
    for (int k = 0; k < top; ++k) fill_f32<T, true>(smem + (size_t)k * F, hidden + ((size_t)r * top + k) * F, F, vec);
    __syncthreads();
    const float sg = shared != nullptr ? (shared_gate != nullptr ? shared_gate[r] : 1.f) : 0.f;
    const int c_end = min(d, (int)(blockIdx.y + 1) * MOE_COLS);
    for (int c = blockIdx.y * MOE_COLS + warp; c < c_end; c += nw) {
        float acc = 0.f;
        // the chosen experts' rows of this column, four dot products in flight at a time
        for (int k0 = 0; k0 < top; k0 += 4) {
            const T* w[4];
            const float* x4[4];
            float wt[4], v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = min(k0 + j, top - 1);
                int e = chosen[(size_t)r * top + k];
                wt[j] = (k0 + j < top && e >= 0 && e < E) ? weights[(size_t)r * top + k] : 0.f;
                e = min(max(e, 0), E - 1);
                w[j] = w_down + ((size_t)e * d + c) * F;
                x4[j] = smem + (size_t)k * F;
            }
            const T* const wc[4] = {w[0], w[1], w[2], w[3]};
            const float* const xc[4] = {x4[0], x4[1], x4[2], x4[3]};
            warp_dots<T, 4>(wc, xc, F, lane, vec, v);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc = fmaf(wt[j], v[j], acc);
        }
        if (lane == 0) {
            if (shared != nullptr) acc = fmaf(sg, to_f32(shared[(size_t)r * lds + c]), acc);
            out[(size_t)r * d + c] = from_f32<T>(acc);
        }
    }
}

template <typename K>
int set_smem(K kernel, size_t bytes, const char* what) {
    if (bytes > 200 * 1024) {
        tis_set_error("%s: %zu bytes of shared memory a CTA (at most 200 KB)", what, bytes);
        return TIS_BAD_SIZE;
    }
    if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return TIS_OK;
}

}  // namespace

TIS_API int tis_moe_route(int dtype, const void* x, int ldx, const float* wr, const float* corr, const float* w_sg,
                          int n, int d, int E, int groups, int keep, int top, float weight_eps, int* chosen,
                          float* weights, float* shared_gate, int score_kind, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || E <= 0 || top <= 0 || top > E || groups < 0 || (groups > 0 && (E % groups || keep <= 0 || keep > groups ||
        top > E / groups * keep)) || (w_sg != nullptr && shared_gate == nullptr)) {
        tis_set_error("moe_route: %d experts, top %d, %d groups of which %d kept", E, top, groups, keep);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * ((size_t)d + 2 * (size_t)E + (size_t)(groups > 0 ? groups : 1));
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_route_kernel<T>, smem, "moe_route");
        if (st != TIS_OK) return st;
        tis_launch(moe_route_kernel<T>, dim3(n), dim3(2 * MOE_THREADS), smem, stream, (const T*)x, ldx, wr, corr, w_sg, d, E,
                   groups, keep, top, weight_eps, chosen, weights, shared_gate, score_kind);
    });
    return tis_check_launch("moe_route");
}

TIS_API int tis_moe_gate_up(int dtype, const void* x, int ldx, const int* chosen, const void* w_gu, void* hidden, int n,
                            int d, int top, int E, int F, int act, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || top <= 0 || E <= 0 || F <= 0) {
        tis_set_error("moe_gate_up: width %d, top %d, %d experts of %d hidden", d, top, E, F);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * (size_t)d;
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_gate_up_kernel<T>, smem, "moe_gate_up");
        if (st != TIS_OK) return st;
        tis_launch(moe_gate_up_kernel<T>, dim3(n * top, (F + MOE_COLS - 1) / MOE_COLS), dim3(MOE_THREADS), smem, stream,
                   (const T*)x, ldx, chosen, (const T*)w_gu, (T*)hidden, d, top, E, F, act);
    });
    return tis_check_launch("moe_gate_up");
}

TIS_API int tis_moe_down(int dtype, const void* hidden, const int* chosen, const float* weights, const void* w_down,
                         const void* shared, int lds, const float* shared_gate, void* out, int n, int d, int top, int E,
                         int F, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || top <= 0 || E <= 0 || F <= 0) {
        tis_set_error("moe_down: width %d, top %d, %d experts of %d hidden", d, top, E, F);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * (size_t)top * F;
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_down_kernel<T>, smem, "moe_down");
        if (st != TIS_OK) return st;
        tis_launch(moe_down_kernel<T>, dim3(n, (d + MOE_COLS - 1) / MOE_COLS), dim3(MOE_THREADS), smem, stream,
                   (const T*)hidden, chosen, weights, (const T*)w_down, (const T*)shared, lds, shared_gate, (T*)out, d, top,
                   E, F);
    });
    return tis_check_launch("moe_down");
}

// ------------------------------------------------------------------------------------------------------------
// Many rows (prompt portions), bfloat16: the rows are sorted by expert on the device and the experts' products run
// as tiles of 64 sorted rows x 64 columns on the tensor cores (mma.sync m16n8k16, operands by cp.async through a ring of
// three stages).  Every expert's rows start on a tile boundary, so a tile belongs to one expert; tile -> expert and
// row -> (token, choice) are tables that the sort kernel writes, and the grid is sized for the worst case
// (pairs / 64 + experts tiles): tiles beyond the last one leave at once.  Nothing comes back to the host.
// ------------------------------------------------------------------------------------------------------------
namespace {

constexpr int GT_ROWS = 64, GT_COLS = 64, GT_BK = 32, GT_STAGES = 3, GT_LD = GT_BK + 8;

// One CTA.  counts -> every expert's first sorted row (a multiple of tile_rows) -> tile_expert; then every pair (token,
// choice) takes the next free place of its expert: sorted_pair[place] = pair, pair_place[pair] = place.  Places that no
// pair takes hold -1.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ chosen, int pairs, int E, int tile_rows, int* __restrict__ sorted_pair, int max_rows,
                int* __restrict__ pair_place, int* __restrict__ tile_expert, int max_tiles) {
    extern __shared__ int sh[];
    int* counts = sh;              // [E]
    int* starts = counts + E;      // [E]
    pdl_launch_dependents();
    const int tid = threadIdx.x, nthr = blockDim.x;
    for (int e = tid; e < E; e += nthr) counts[e] = 0;
    pdl_wait();
    for (int i = tid; i < max_rows; i += nthr) sorted_pair[i] = -1;
    __syncthreads();
    for (int p = tid; p < pairs; p += nthr) {
        const int e = chosen[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            starts[e] = tile * tile_rows;
            const int tiles = (counts[e] + tile_rows - 1) / tile_rows;
            for (int t = 0; t < tiles && tile < max_tiles; ++t) tile_expert[tile++] = e;
        }
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
    }
    __syncthreads();
    for (int e = tid; e < E; e += nthr) counts[e] = 0;      // now the next free place of every expert
    __syncthreads();
    for (int p = tid; p < pairs; p += nthr) {
        const int e = chosen[p];
        if (e < 0 || e >= E) { pair_place[p] = -1; continue; }
        const int place = starts[e] + atomicAdd(&counts[e], 1);
        if (place < max_rows) { sorted_pair[place] = p; pair_place[p] = place; } else pair_place[p] = -1;
    }
}

__device__ __forceinline__ void g_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void g_mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void g_cp_async16(void* smem, const void* gmem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem));
}

// C[tile rows][n0 .. n0 + 64) = A . W[e]^T over K.  GATED: W[e] holds N gate rows and then N up rows, and C = silu(gate) *
// up; else W[e] holds N rows.  GATHER: row i of the tile is row sorted_pair[.] / top of A (a token's input; places
// without a pair: zeros); else row i of the tile is row tile * 64 + i of A (the sorted hidden rows).  act >= 0 (not GATED):
// C = act(A . W[e]^T), the first product of units without a gate.
template <bool GATED, bool GATHER>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ sorted_pair, int top,
                   const int* __restrict__ tile_expert, const bf16* __restrict__ W, size_t expert_stride,
                   bf16* __restrict__ C, int ldc, int N, int K, int act) {
    constexpr int BROWS = GATED ? 2 * GT_COLS : GT_COLS;
    __shared__ __align__(16) bf16 As[GT_STAGES][GT_ROWS][GT_LD];
    __shared__ __align__(16) bf16 Bs[GT_STAGES][BROWS][GT_LD];
    __shared__ int src_row[GT_ROWS];
    pdl_launch_dependents();
    const int tile = blockIdx.x, n0 = blockIdx.y * GT_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    const int e = tile_expert[tile];
    if (e < 0) return;
    if (tid < GT_ROWS) {
        int r = tile * GT_ROWS + tid;
        if (GATHER) { const int p = sorted_pair[r]; r = p >= 0 ? p / top : -1; }
        src_row[tid] = r;
    }
    __syncthreads();
    const bf16* We = W + (size_t)e * expert_stride;
    auto load_stage = [&](int s, int k0) {
        // A: 64 rows x 4 chunks of 8 elements; B: BROWS rows x 4 chunks
        for (int idx = tid; idx < GT_ROWS * (GT_BK / 8); idx += 128) {
            const int i = idx >> 2, c = idx & 3;
            const int r = src_row[i];
            bf16* dst = &As[s][i][c * 8];
            if (r >= 0) g_cp_async16(dst, A + (size_t)r * lda + k0 + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        for (int idx = tid; idx < BROWS * (GT_BK / 8); idx += 128) {
            const int j = idx >> 2, c = idx & 3;
            const int n = n0 + (j & (GT_COLS - 1));
            bf16* dst = &Bs[s][j][c * 8];
            if (n < N) g_cp_async16(dst, We + ((size_t)(GATED && j >= GT_COLS ? N : 0) + n) * K + k0 + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // the four warps as 2 x 2: a warp owns 32 rows x 32 columns (of the gate and of the up matrix), so that an operand
    // fragment it loads serves two products
    const int wm = warp >> 1, wn = warp & 1;
    float acc[GATED ? 2 : 1][2][4][4];
#pragma unroll
    for (int h = 0; h < (GATED ? 2 : 1); ++h)
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int n = 0; n < 4; ++n) { acc[h][mi][n][0] = acc[h][mi][n][1] = acc[h][mi][n][2] = acc[h][mi][n][3] = 0.f; }
    const int nk = K / GT_BK;
#pragma unroll
    for (int s = 0; s < GT_STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s * GT_BK);
        else asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(GT_STAGES - 2));
        __syncthreads();
        const int nxt = kt + GT_STAGES - 1;
        if (nxt < nk) load_stage(nxt % GT_STAGES, nxt * GT_BK);
        else asm volatile("cp.async.commit_group;\n" ::);
        const int s = kt % GT_STAGES;
#pragma unroll
        for (int kk = 0; kk < GT_BK / 16; ++kk) {
            unsigned a[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                g_ldmatrix_x4(a[mi], &As[s][wm * 32 + mi * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][kk * 16 + 8 * (lane >> 4)]);
#pragma unroll
            for (int h = 0; h < (GATED ? 2 : 1); ++h) {
#pragma unroll
                for (int n2 = 0; n2 < 2; ++n2) {
                    unsigned b[4];
                    g_ldmatrix_x4(b, &Bs[s][h * GT_COLS + wn * 32 + n2 * 16 + (lane & 7) + 8 * (lane >> 4)][kk * 16 + 8 * ((lane >> 3) & 1)]);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        g_mma_bf16(acc[h][mi][2 * n2], a[mi], b[0], b[1]);
                        g_mma_bf16(acc[h][mi][2 * n2 + 1], a[mi], b[2], b[3]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const size_t row = (size_t)tile * GT_ROWS + wm * 32 + mi * 16 + g + 8 * half;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const int col = n0 + wn * 32 + n * 8 + 2 * t4;
                float v0 = acc[0][mi][n][2 * half], v1 = acc[0][mi][n][2 * half + 1];
                if (GATED) {
                    v0 = v0 / (1.f + __expf(-v0)) * acc[GATED ? 1 : 0][mi][n][2 * half];
                    v1 = v1 / (1.f + __expf(-v1)) * acc[GATED ? 1 : 0][mi][n][2 * half + 1];
                } else if (act >= 0) {
                    v0 = unit_act(v0, act);
                    v1 = unit_act(v1, act);
                }
                if (col + 1 < N) *reinterpret_cast<__nv_bfloat162*>(C + row * ldc + col) = __floats2bfloat162_rn(v0, v1);
                else if (col < N) C[row * ldc + col] = __float2bfloat16_rn(v0);
            }
        }
    }
}

// out[r][c] = sum_k weights[r][k] * y[pair_place[r * top + k]][c]  (+ shared_gate[r] * shared[r][c])
__global__ void __launch_bounds__(256)
moe_combine_kernel(const bf16* __restrict__ y, int ldy, const int* __restrict__ pair_place, const float* __restrict__ weights,
                   const bf16* __restrict__ shared, int lds, const float* __restrict__ shared_gate, bf16* __restrict__ out,
                   int d, int top) {
    pdl_launch_dependents();
    const int r = blockIdx.x;
    pdl_wait();
    const float sg = shared != nullptr ? (shared_gate != nullptr ? shared_gate[r] : 1.f) : 0.f;
    for (int c = threadIdx.x * 2; c < d; c += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
        for (int k = 0; k < top; ++k) {
            const int place = pair_place[(size_t)r * top + k];
            if (place < 0) continue;
            const float w = weights[(size_t)r * top + k];
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(y + (size_t)place * ldy + c);
            a0 = fmaf(w, __bfloat162float(v.x), a0);
            a1 = fmaf(w, __bfloat162float(v.y), a1);
        }
        if (shared != nullptr) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(shared + (size_t)r * lds + c);
            a0 = fmaf(sg, __bfloat162float(v.x), a0);
            a1 = fmaf(sg, __bfloat162float(v.y), a1);
        }
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)r * d + c) = __floats2bfloat162_rn(a0, a1);
    }
}

}  // namespace

// The sort and the weighted sum, for the tile kernels of this file and of moe_tc.cu.
int tis_moe_sort_launch(const int* chosen, int pairs, int E, int tile_rows, int* sorted_pair, int max_rows, int* pair_place,
                        int* tile_expert, int max_tiles, cudaStream_t stream) {
    tis_launch(moe_sort_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * (size_t)E, stream, chosen, pairs, E, tile_rows,
               sorted_pair, max_rows, pair_place, tile_expert, max_tiles);
    return tis_check_launch("moe_sort");
}

int tis_moe_combine_launch(const void* y, int ldy, const int* pair_place, const float* weights, const void* shared, int lds,
                           const float* shared_gate, void* out, int n, int d, int top, cudaStream_t stream) {
    tis_launch(moe_combine_kernel, dim3(n), dim3(256), 0, stream, (const bf16*)y, ldy, pair_place, weights, (const bf16*)shared,
               lds, shared_gate, (bf16*)out, d, top);
    return tis_check_launch("moe_combine");
}

// Tiles of 64 sorted rows that `pairs` (token, choice) pairs over E experts can need at most.
TIS_API int tis_moe_grouped_tiles(int pairs, int E) { return (pairs + GT_ROWS - 1) / GT_ROWS + E; }

// The experts' products for many rows in bfloat16.  x (n, d) with row stride ldx; w_gu (E, 2, F, d), or (E, F, d) with
// act >= 0 (units without a gate); w_down (E, d, F);
// scratch: sorted_pair and hidden / y rows for tis_moe_grouped_tiles(n * top, E) * 64 places, pair_place n * top,
// tile_expert that many tiles.  d and F multiples of 32; ldx, lds multiples of 8 and even; operands 16-byte aligned.
TIS_API int tis_moe_grouped(const void* x, int ldx, const int* chosen, const float* weights, const void* w_gu,
                            const void* w_down, const void* shared, int lds, const float* shared_gate, void* out,
                            int* sorted_pair, int* pair_place, int* tile_expert, void* hidden, void* y, int n, int d,
                            int top, int E, int F, int act, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || F <= 0 || d % GT_BK || F % GT_BK || ldx % 8 || lds % 2 || E <= 0 || E > 4096 || top <= 0 ||
        ((uintptr_t)x | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)hidden | (uintptr_t)y) % 16 ||
        ((uintptr_t)shared | (uintptr_t)out) % 4) {
        tis_set_error("moe_grouped: width %d and hidden %d must be multiples of %d, operands aligned (%d experts, top %d)",
                      d, F, GT_BK, E, top);
        return TIS_BAD_SIZE;
    }
    const int pairs = n * top, tiles = tis_moe_grouped_tiles(pairs, E);
    int st = tis_moe_sort_launch(chosen, pairs, E, GT_ROWS, sorted_pair, tiles * GT_ROWS, pair_place, tile_expert, tiles, stream);
    if (st != TIS_OK) return st;
    if (act >= 0)
        tis_launch(moe_grouped_kernel<false, true>, dim3(tiles, (F + GT_COLS - 1) / GT_COLS), dim3(128), 0, stream,
                   (const bf16*)x, ldx, (const int*)sorted_pair, top, (const int*)tile_expert, (const bf16*)w_gu, (size_t)F * d,
                   (bf16*)hidden, F, F, d, act);
    else
        tis_launch(moe_grouped_kernel<true, true>, dim3(tiles, (F + GT_COLS - 1) / GT_COLS), dim3(128), 0, stream,
                   (const bf16*)x, ldx, (const int*)sorted_pair, top, (const int*)tile_expert, (const bf16*)w_gu,
                   (size_t)2 * F * d, (bf16*)hidden, F, F, d, -1);
    st = tis_check_launch("moe_grouped_gate_up");
    if (st != TIS_OK) return st;
    tis_launch(moe_grouped_kernel<false, false>, dim3(tiles, (d + GT_COLS - 1) / GT_COLS), dim3(128), 0, stream,
               (const bf16*)hidden, F, (const int*)sorted_pair, top, (const int*)tile_expert, (const bf16*)w_down, (size_t)d * F,
               (bf16*)y, d, d, F, -1);
    st = tis_check_launch("moe_grouped_down");
    if (st != TIS_OK) return st;
    return tis_moe_combine_launch(y, d, pair_place, weights, shared, lds, shared_gate, out, n, d, top, stream);
}
