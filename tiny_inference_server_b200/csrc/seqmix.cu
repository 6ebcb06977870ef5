// Kernels of mixers that are not plain rotary attention:
//   * a short causal convolution over time on each channel, with the last inputs of a request kept in its state;
//   * the step between the projections and the cache of an attention whose queries and keys are normalised as a
//     whole and whose values are mixed with another layer's: norm, mix, write into the pages;
//   * attention over a window of the paged cache with keys and values of different widths, a bias on the scores
//     that grows with the logarithm of the distance, and a sigmoid gate on the output;
//   * the delta rule with a decay per head and key channel, a recurrence over a matrix state per head.
// Everything is computed in 32-bit; T is the storage type of activations and pages.
//
// Rows of a step: row r belongs to request slot row_slot[r] (negative: padding) at positions[r]; the rows of a
// request are consecutive and in order, row_last[r] is the last row of r's request in this step.
#include "common.cuh"

// ------------------------------------------------------------------------------------------------------------
// y[r, c] = (residual ? x[r, c] : 0) + bias[c] + sum_j w[j, c] * x(t - taps + 1 + j)[c], optionally through silu (the
// weights lie tap by tap: [taps][C]; bias null: none).
// x(t') of a position before this step's rows of the request comes from the request's state, which holds its
// last taps-1 inputs (oldest first, zero before the start of the sequence) and is brought up to date here.
//
// A thread owns one (row, channel).  The state of a (request, channel) is read and written by one thread only:
// the thread of the request's first row in this step computes the first taps-1 rows of the request, which are the
// ones that need the state, and then writes the new state; the threads of those rows do nothing.
// ------------------------------------------------------------------------------------------------------------
constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, float* __restrict__ state,
                   size_t state_stride, T* __restrict__ out, int ldo, const int* __restrict__ row_slot,
                   const int* __restrict__ row_last, int n, int C, int taps, int residual, int act_silu,
                   const float* __restrict__ bias) {
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int hist = taps - 1;
    int back = 0;
    while (back < hist && r - back - 1 >= 0 && row_slot[r - back - 1] == slot) ++back;
    if (back > 0 && back < hist) return;              // computed by the thread of the request's first row
    float wt[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)j * C + c] : 0.f;
    const float b0 = bias != nullptr ? bias[c] : 0.f;
    pdl_wait();
    if (back == hist) {                               // every input is a row of this step (or there is no history)
        float acc = 0.f, cur = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < taps) {
                cur = to_f32(x[(size_t)(r - hist + j) * ldx + c]);
                acc = fmaf(wt[j], cur, acc);
            }
        }
        acc += b0;
        if (residual) acc += cur;
        if (act_silu) acc = acc / (1.f + expf(-acc));
        out[(size_t)r * ldo + c] = from_f32<T>(acc);
        return;
    }
    // the first row of a request in this step
    const int rows = row_last[r] - r + 1;
    float* st = state + (size_t)slot * state_stride;
    float h[CONV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) h[k] = k < hist ? st[(size_t)k * C + c] : 0.f;
    const int mine = rows < hist ? rows : hist;
    for (int i = 0; i < mine; ++i) {
        const float cur = to_f32(x[(size_t)(r + i) * ldx + c]);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS; ++k)
            if (k < hist) acc = fmaf(wt[k], h[k], acc);
        acc = fmaf(wt[hist], cur, acc) + b0;
        if (residual) acc += cur;
        if (act_silu) acc = acc / (1.f + expf(-acc));
        out[(size_t)(r + i) * ldo + c] = from_f32<T>(acc);
#pragma unroll
        for (int k = 0; k + 1 < CONV_MAX_TAPS; ++k)
            if (k + 1 < hist) h[k] = h[k + 1];
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS; ++k)
            if (k == hist - 1) h[k] = cur;
    }
    if (rows > hist) {
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS; ++k)
            if (k < hist) h[k] = to_f32(x[(size_t)(r + rows - hist + k) * ldx + c]);
    }
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k)
        if (k < hist) st[(size_t)k * C + c] = h[k];
}

// The same for channel counts and row strides that are multiples of a 16-byte vector: a thread owns a (row, vector
// of channels) and the taps are a template parameter, so that weights and history stay in registers.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
causal_conv_vec_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, float* __restrict__ state,
                       size_t state_stride, T* __restrict__ out, int ldo, const int* __restrict__ row_slot,
                       const int* __restrict__ row_last, int n, int C, int residual, int act_silu,
                       const float* __restrict__ bias) {
    constexpr int N = Vec16<T>::N, HIST = TAPS - 1;
    pdl_launch_dependents();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * N;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int slot = row_slot[r];
    if (slot < 0) return;
    int back = 0;
    while (back < HIST && r - back - 1 >= 0 && row_slot[r - back - 1] == slot) ++back;
    if (back > 0 && back < HIST) return;              // computed by the thread of the request's first row
    float wt[N][TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j)
#pragma unroll
        for (int e = 0; e < N; e += 4) {
            const float4 v = *reinterpret_cast<const float4*>(w + (size_t)j * C + c + e);
            wt[e][j] = v.x; wt[e + 1][j] = v.y; wt[e + 2][j] = v.z; wt[e + 3][j] = v.w;
        }
    float b0[N];
#pragma unroll
    for (int e = 0; e < N; ++e) b0[e] = bias != nullptr ? bias[c + e] : 0.f;
    pdl_wait();
    auto finish = [&](float (&acc)[N], const float (&cur)[N], size_t row) {
#pragma unroll
        for (int e = 0; e < N; ++e) {
            acc[e] += b0[e];
            if (residual) acc[e] += cur[e];
            if (act_silu) acc[e] = acc[e] / (1.f + expf(-acc[e]));
        }
        Vec16<T>::store(out + row * ldo + c, acc);
    };
    if (back == HIST) {
        float acc[N], cur[N];
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] = 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            Vec16<T>::load(x + (size_t)(r - HIST + j) * ldx + c, cur);
#pragma unroll
            for (int e = 0; e < N; ++e) acc[e] = fmaf(wt[e][j], cur[e], acc[e]);
        }
        finish(acc, cur, (size_t)r);
        return;
    }
    const int rows = row_last[r] - r + 1;
    float* st = state + (size_t)slot * state_stride;
    float h[HIST > 0 ? HIST : 1][N];
#pragma unroll
    for (int k = 0; k < HIST; ++k)
#pragma unroll
        for (int e = 0; e < N; ++e) h[k][e] = st[(size_t)k * C + c + e];
    const int mine = rows < HIST ? rows : HIST;
    for (int i = 0; i < mine; ++i) {
        float acc[N], cur[N];
        Vec16<T>::load(x + (size_t)(r + i) * ldx + c, cur);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            float a = 0.f;                              // the taps in the order of the other path: bit-equal results
#pragma unroll
            for (int k = 0; k < HIST; ++k) a = fmaf(wt[e][k], h[k][e], a);
            acc[e] = fmaf(wt[e][HIST], cur[e], a);
        }
#pragma unroll
        for (int k = 0; k + 1 < HIST; ++k)
#pragma unroll
            for (int e = 0; e < N; ++e) h[k][e] = h[k + 1][e];
        if (HIST > 0) {
#pragma unroll
            for (int e = 0; e < N; ++e) h[HIST - 1][e] = cur[e];
        }
        finish(acc, cur, (size_t)(r + i));
    }
    if (rows > HIST) {
#pragma unroll
        for (int k = 0; k < HIST; ++k) Vec16<T>::load(x + (size_t)(r + rows - HIST + k) * ldx + c, h[k]);
    }
#pragma unroll
    for (int k = 0; k < HIST; ++k)
#pragma unroll
        for (int e = 0; e < N; ++e) st[(size_t)k * C + c + e] = h[k][e];
}

template <typename T, int TAPS>
static void launch_causal_conv_vec(const T* x, int ldx, const float* w, float* state, size_t state_stride, T* out, int ldo,
                                   const int* row_slot, const int* row_last, int n, int C, int residual, int act_silu,
                                   const float* bias, cudaStream_t stream) {
    constexpr int N = Vec16<T>::N;
    const int vecs = C / N;
    const int threads = vecs >= 128 ? 128 : (vecs + 31) / 32 * 32;
    tis_launch(causal_conv_vec_kernel<T, TAPS>, dim3((vecs + threads - 1) / threads, n), dim3(threads), 0, stream, x, ldx, w,
               state, state_stride, out, ldo, row_slot, row_last, n, C, residual, act_silu, bias);
}

TIS_API int tis_causal_conv(int dtype, const void* x, int ldx, const float* w, float* state, size_t state_stride,
                            void* out, int ldo, const int* row_slot, const int* row_last, int n, int C, int taps,
                            int residual, int act_silu, const float* bias, cudaStream_t stream) {
    if (n <= 0 || C <= 0) return TIS_OK;
    if (taps < 1 || taps > CONV_MAX_TAPS) {
        tis_set_error("causal_conv: %d taps; this kernel takes 1..%d", taps, CONV_MAX_TAPS);
        return TIS_BAD_SIZE;
    }
    if (x == out) {
        tis_set_error("causal_conv: a row reads the rows before it, so the result needs a place of its own");
        return TIS_BAD_SIZE;
    }
    const int per = dtype == TIS_BF16 ? 8 : 4;
    if (taps >= 2 && taps <= 5 && C % per == 0 && ldx % per == 0 && ldo % per == 0 &&
        ((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) % 16 == 0) {
#define TIS_CONV_CASE(K)                                                                                               \
    case K:                                                                                                            \
        TIS_DISPATCH_DTYPE(dtype, T, launch_causal_conv_vec<T, K>((const T*)x, ldx, w, state, state_stride, (T*)out,   \
            ldo, row_slot, row_last, n, C, residual, act_silu, bias, stream));                                               \
        break;
        switch (taps) {
            TIS_CONV_CASE(2)
            TIS_CONV_CASE(3)
            TIS_CONV_CASE(4)
            TIS_CONV_CASE(5)
        }
#undef TIS_CONV_CASE
        return tis_check_launch("causal_conv");
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(causal_conv_kernel<T>, dim3((C + 127) / 128, n), dim3(128), 0, stream, (const T*)x, ldx, w, state,
                   state_stride, (T*)out, ldo, row_slot, row_last, n, C, taps, residual, act_silu, bias));
    return tis_check_launch("causal_conv");
}

// ------------------------------------------------------------------------------------------------------------
// Between the projections and the cache.  A row of `qkv` holds nq query, nk key and nv value elements (all heads).
//   queries: q * rsqrt(mean(q^2) + eps) * wq over all nq elements at once, in place (wq null: left as they are);
//   keys: the same with wk over nk elements, written into the row's page;
//   values: (1 - lambda) * v + lambda * v_other (v_other null: v itself), written into the row's page.
// Pages: element (page, kv head, position in the page, i) of the keys at k_pages + page * k_page_stride +
// head * k_head_stride + position * k_dim + i; the values likewise.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
norm_mix_store_kernel(T* __restrict__ qkv, int ld, int nq, int nk, int nv, const float* __restrict__ wq,
                      const float* __restrict__ wk, float eps, const T* __restrict__ v_other, int ld_other,
                      const float* __restrict__ lambda, T* __restrict__ k_pages, size_t k_page_stride,
                      size_t k_head_stride, T* __restrict__ v_pages, size_t v_page_stride, size_t v_head_stride,
                      int kv_heads, int page_size, int num_pages, const int* __restrict__ block_table, int bt_stride,
                      const int* __restrict__ positions, const int* __restrict__ row_slot, int* __restrict__ fault) {
    __shared__ float red[33];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    pdl_wait();
    T* row = qkv + (size_t)r * ld;
    float sq = 0.f, sk = 0.f;
    if (wq != nullptr)
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = to_f32(row[i]); sq += v * v; }
    if (wk != nullptr)
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = to_f32(row[nq + i]); sk += v * v; }
    if (wq != nullptr) {
        sq = block_sum(sq, red);
        const float f = rsqrtf(sq / (float)nq + eps);
        for (int i = threadIdx.x; i < nq; i += blockDim.x) row[i] = from_f32<T>(to_f32(row[i]) * f * wq[i]);
    }
    float fk = 1.f;
    if (wk != nullptr) {
        sk = block_sum(sk, red);
        fk = rsqrtf(sk / (float)nk + eps);
    }
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(fault, 3);
        return;
    }
    const int in_page = pos % page_size;
    const int k_dim = nk / kv_heads, v_dim = nv / kv_heads;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int head = i / k_dim, e = i - head * k_dim;
        const float v = to_f32(row[nq + i]) * fk * (wk != nullptr ? wk[i] : 1.f);
        k_pages[(size_t)page * k_page_stride + (size_t)head * k_head_stride + (size_t)in_page * k_dim + e] = from_f32<T>(v);
    }
    const float lam = (v_other != nullptr && lambda != nullptr) ? lambda[0] : 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int head = i / v_dim, e = i - head * v_dim;
        float v = to_f32(row[nq + nk + i]);
        if (v_other != nullptr) v = (1.f - lam) * v + lam * to_f32(v_other[(size_t)r * ld_other + i]);
        v_pages[(size_t)page * v_page_stride + (size_t)head * v_head_stride + (size_t)in_page * v_dim + e] = from_f32<T>(v);
    }
}

// The same with 16-byte vectors, for widths and strides that are multiples of a vector.
template <typename T>
__global__ void __launch_bounds__(256)
norm_mix_store_vec_kernel(T* __restrict__ qkv, int ld, int nq, int nk, int nv, const float* __restrict__ wq,
                          const float* __restrict__ wk, float eps, const T* __restrict__ v_other, int ld_other,
                          const float* __restrict__ lambda, T* __restrict__ k_pages, size_t k_page_stride,
                          size_t k_head_stride, T* __restrict__ v_pages, size_t v_page_stride, size_t v_head_stride,
                          int kv_heads, int page_size, int num_pages, const int* __restrict__ block_table, int bt_stride,
                          const int* __restrict__ positions, const int* __restrict__ row_slot, int* __restrict__ fault) {
    constexpr int N = Vec16<T>::N;
    __shared__ float red[33];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    pdl_wait();
    T* row = qkv + (size_t)r * ld;
    float sq = 0.f, sk = 0.f;
    float x[N];
    if (wq != nullptr)
        for (int i = threadIdx.x * N; i < nq; i += blockDim.x * N) {
            Vec16<T>::load(row + i, x);
#pragma unroll
            for (int e = 0; e < N; ++e) sq = fmaf(x[e], x[e], sq);
        }
    if (wk != nullptr)
        for (int i = threadIdx.x * N; i < nk; i += blockDim.x * N) {
            Vec16<T>::load(row + nq + i, x);
#pragma unroll
            for (int e = 0; e < N; ++e) sk = fmaf(x[e], x[e], sk);
        }
    if (wq != nullptr) {
        sq = block_sum(sq, red);
        const float f = rsqrtf(sq / (float)nq + eps);
        for (int i = threadIdx.x * N; i < nq; i += blockDim.x * N) {
            Vec16<T>::load(row + i, x);
#pragma unroll
            for (int e = 0; e < N; ++e) x[e] = x[e] * f * wq[i + e];
            Vec16<T>::store(row + i, x);
        }
    }
    float fk = 1.f;
    if (wk != nullptr) {
        sk = block_sum(sk, red);
        fk = rsqrtf(sk / (float)nk + eps);
    }
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(fault, 3);
        return;
    }
    const int in_page = pos % page_size;
    const int k_dim = nk / kv_heads, v_dim = nv / kv_heads;
    for (int i = threadIdx.x * N; i < nk; i += blockDim.x * N) {
        const int head = i / k_dim, e0 = i - head * k_dim;
        Vec16<T>::load(row + nq + i, x);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] = x[e] * fk * (wk != nullptr ? wk[i + e] : 1.f);
        Vec16<T>::store(k_pages + (size_t)page * k_page_stride + (size_t)head * k_head_stride + (size_t)in_page * k_dim + e0, x);
    }
    const float lam = (v_other != nullptr && lambda != nullptr) ? lambda[0] : 0.f;
    for (int i = threadIdx.x * N; i < nv; i += blockDim.x * N) {
        const int head = i / v_dim, e0 = i - head * v_dim;
        Vec16<T>::load(row + nq + nk + i, x);
        if (v_other != nullptr) {
            float y[N];
            Vec16<T>::load(v_other + (size_t)r * ld_other + i, y);
#pragma unroll
            for (int e = 0; e < N; ++e) x[e] = (1.f - lam) * x[e] + lam * y[e];
        }
        Vec16<T>::store(v_pages + (size_t)page * v_page_stride + (size_t)head * v_head_stride + (size_t)in_page * v_dim + e0, x);
    }
}

TIS_API int tis_norm_mix_store(int dtype, void* qkv, int ld, int nq, int nk, int nv, const float* wq, const float* wk,
                               float eps, const void* v_other, int ld_other, const float* lambda, void* k_pages,
                               size_t k_page_stride, size_t k_head_stride, void* v_pages, size_t v_page_stride,
                               size_t v_head_stride, int kv_heads, int page_size, int num_pages,
                               const int* block_table, int bt_stride, const int* positions, const int* row_slot,
                               int* fault, int n, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (kv_heads <= 0 || nk % kv_heads || nv % kv_heads || page_size <= 0) {
        tis_set_error("norm_mix_store: %d key and %d value elements for %d kv heads, page size %d", nk, nv, kv_heads,
                      page_size);
        return TIS_BAD_SIZE;
    }
    const int per = dtype == TIS_BF16 ? 8 : 4;
    const int kd = nk / kv_heads, vd = nv / kv_heads;
    if (nq % per == 0 && kd % per == 0 && vd % per == 0 && ld % per == 0 && (v_other == nullptr || ld_other % per == 0) &&
        k_page_stride % per == 0 && k_head_stride % per == 0 && v_page_stride % per == 0 && v_head_stride % per == 0 &&
        ((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)v_other) % 16 == 0) {
        TIS_DISPATCH_DTYPE(dtype, T,
            tis_launch(norm_mix_store_vec_kernel<T>, dim3(n), dim3(256), 0, stream, (T*)qkv, ld, nq, nk, nv, wq, wk, eps,
                       (const T*)v_other, ld_other, lambda, (T*)k_pages, k_page_stride, k_head_stride, (T*)v_pages,
                       v_page_stride, v_head_stride, kv_heads, page_size, num_pages, block_table, bt_stride, positions,
                       row_slot, fault));
        return tis_check_launch("norm_mix_store");
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(norm_mix_store_kernel<T>, dim3(n), dim3(256), 0, stream, (T*)qkv, ld, nq, nk, nv, wq, wk, eps,
                   (const T*)v_other, ld_other, lambda, (T*)k_pages, k_page_stride, k_head_stride, (T*)v_pages,
                   v_page_stride, v_head_stride, kv_heads, page_size, num_pages, block_table, bt_stride, positions,
                   row_slot, fault));
    return tis_check_launch("norm_mix_store");
}

// ------------------------------------------------------------------------------------------------------------
// Between the projections and the cache of attention whose heads carry several score maps over the same values.
// A row of `qkv` holds H * M query runs, G * M key runs (`dim` elements each: head by head, map by map) and G value
// runs of `vdim` elements.  `bias` (all of these, in the row's order; null: none) is added first.  Every query and key
// run is divided by its root mean square (eps inside the root) and multiplied by wq / wk (`dim` weights, the same for
// every run; null: left as it is).  Queries are then multiplied by 1 + coef * ln(floor((pos + 1) / every) + 1)
// (every <= 0: not).  Keys and values go to the row's page: a key row of a kv head is its M runs side by side.
// Queries go to q_out as H * M query heads of the key row's whole width M * dim: run (h, m) fills the m-th stretch
// of `dim` elements of head h * M + m and the other stretches are zero, so that a product with a key row meets only
// the key's run of the same map.  A CTA a row, a warp a run.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_store_kernel(const T* __restrict__ qkv, int ld, int H, int G, int M, int dim, int vdim,
                       const float* __restrict__ bias, const float* __restrict__ wq, const float* __restrict__ wk,
                       float eps, float temp_coef, int temp_every, T* __restrict__ q_out, int ldq,
                       T* __restrict__ k_pages, size_t k_page_stride, size_t k_head_stride, T* __restrict__ v_pages,
                       size_t v_page_stride, size_t v_head_stride, int page_size, int num_pages,
                       const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                       const int* __restrict__ row_slot, int* __restrict__ fault) {
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (pos < 0 || page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(fault, 7);
        return;
    }
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
    const int in_page = pos % page_size;
    const int q_runs = H * M, k_runs = G * M, kw = M * dim;
    pdl_wait();
    const T* row = qkv + (size_t)r * ld;
    for (int run = warp; run < q_runs + k_runs; run += nwarps) {
        const bool is_q = run < q_runs;
        const int at = run * dim;                       // queries first, keys behind them: runs are contiguous
        const float* w = is_q ? wq : wk;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float v = to_f32(row[at + i]) + (bias != nullptr ? bias[at + i] : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        float f = w != nullptr ? rsqrtf(ss / (float)dim + eps) : 1.f;
        if (is_q) f *= temp;
        const int m = run % M;
        if (is_q) {
            T* dst = q_out + (size_t)r * ldq + (size_t)run * kw;
            for (int i = lane; i < kw; i += 32) {
                const int e = i - m * dim;
                float v = 0.f;
                if (e >= 0 && e < dim)
                    v = (to_f32(row[at + e]) + (bias != nullptr ? bias[at + e] : 0.f)) * f * (w != nullptr ? w[e] : 1.f);
                dst[i] = from_f32<T>(v);
            }
        } else {
            const int kvh = (run - q_runs) / M;
            T* dst = k_pages + (size_t)page * k_page_stride + (size_t)kvh * k_head_stride + (size_t)in_page * kw + m * dim;
            for (int i = lane; i < dim; i += 32) {
                const float v = (to_f32(row[at + i]) + (bias != nullptr ? bias[at + i] : 0.f)) * f * (w != nullptr ? w[i] : 1.f);
                dst[i] = from_f32<T>(v);
            }
        }
    }
    const int v_at = (q_runs + k_runs) * dim;
    for (int i = threadIdx.x; i < G * vdim; i += blockDim.x) {
        const int kvh = i / vdim, e = i - kvh * vdim;
        const float v = to_f32(row[v_at + i]) + (bias != nullptr ? bias[v_at + i] : 0.f);
        v_pages[(size_t)page * v_page_stride + (size_t)kvh * v_head_stride + (size_t)in_page * vdim + e] = from_f32<T>(v);
    }
}

// The same with 16-byte vectors, for runs, value rows and strides that are multiples of a vector and runs of
// `lanes` = dim / vector lanes, a power of two up to 32: `lanes` neighbouring lanes hold a run in registers (one pass
// over the input), 256 / lanes runs at a time.
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_store_vec_kernel(const T* __restrict__ qkv, int ld, int H, int G, int M, int dim, int vdim,
                           const float* __restrict__ bias, const float* __restrict__ wq, const float* __restrict__ wk,
                           float eps, float temp_coef, int temp_every, T* __restrict__ q_out, int ldq,
                           T* __restrict__ k_pages, size_t k_page_stride, size_t k_head_stride, T* __restrict__ v_pages,
                           size_t v_page_stride, size_t v_head_stride, int page_size, int num_pages,
                           const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                           const int* __restrict__ row_slot, int* __restrict__ fault) {
    constexpr int N = Vec16<T>::N;
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    if (pos < 0 || page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(fault, 7);
        return;
    }
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
    const int in_page = pos % page_size;
    const int q_runs = H * M, k_runs = G * M, kw = M * dim, runs = q_runs + k_runs;
    const int lanes = dim / N, groups = blockDim.x / lanes;
    const int group = threadIdx.x / lanes, e0 = (threadIdx.x % lanes) * N;
    pdl_wait();
    const T* row = qkv + (size_t)r * ld;
    float x[N], zero[N];
#pragma unroll
    for (int e = 0; e < N; ++e) zero[e] = 0.f;
    for (int base = 0; base < runs; base += groups) {       // every lane of a warp stays in the loop for the shuffles
        const int run = base + group;
        const bool live = run < runs;
        const bool is_q = run < q_runs;
        const int at = run * dim + e0;
        float ss = 0.f;
        if (live) {
            Vec16<T>::load(row + at, x);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                if (bias != nullptr) x[e] += bias[at + e];
                ss = fmaf(x[e], x[e], ss);
            }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (!live) continue;
        const float* w = is_q ? wq : wk;
        float f = w != nullptr ? rsqrtf(ss / (float)dim + eps) : 1.f;
        if (is_q) f *= temp;
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] = x[e] * f * (w != nullptr ? w[e0 + e] : 1.f);
        const int m = run % M;
        if (is_q) {
            T* dst = q_out + (size_t)r * ldq + (size_t)run * kw + e0;
            for (int mm = 0; mm < M; ++mm) Vec16<T>::store(dst + mm * dim, mm == m ? x : zero);
        } else {
            const int kvh = (run - q_runs) / M;
            Vec16<T>::store(k_pages + (size_t)page * k_page_stride + (size_t)kvh * k_head_stride + (size_t)in_page * kw +
                            m * dim + e0, x);
        }
    }
    const int v_at = runs * dim;
    for (int i = threadIdx.x * N; i < G * vdim; i += blockDim.x * N) {
        const int kvh = i / vdim, e = i - kvh * vdim;
        Vec16<T>::load(row + v_at + i, x);
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < N; ++j) x[j] += bias[v_at + i + j];
        }
        Vec16<T>::store(v_pages + (size_t)page * v_page_stride + (size_t)kvh * v_head_stride + (size_t)in_page * vdim + e, x);
    }
}

TIS_API int tis_head_norm_store(int dtype, const void* qkv, int ld, int H, int G, int M, int dim, int vdim,
                                const float* bias, const float* wq, const float* wk, float eps, float temp_coef,
                                int temp_every, void* q_out, int ldq, void* k_pages, size_t k_page_stride,
                                size_t k_head_stride, void* v_pages, size_t v_page_stride, size_t v_head_stride,
                                int page_size, int num_pages, const int* block_table, int bt_stride,
                                const int* positions, const int* row_slot, int* fault, int n, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (H <= 0 || G <= 0 || M <= 0 || dim <= 0 || vdim <= 0 || page_size <= 0 || ld < ((H + G) * M * dim + G * vdim) ||
        ldq < H * M * M * dim) {
        tis_set_error("head_norm_store: %d query heads, %d kv heads, %d maps of %d elements, value width %d, page size %d, "
                      "row lengths %d in and %d out", H, G, M, dim, vdim, page_size, ld, ldq);
        return TIS_BAD_SIZE;
    }
    const int per = dtype == TIS_BF16 ? 8 : 4;
    const int lanes = dim / per;
    if (dim % per == 0 && lanes <= 32 && (lanes & (lanes - 1)) == 0 && vdim % per == 0 && ld % per == 0 && ldq % per == 0 &&
        k_page_stride % per == 0 && k_head_stride % per == 0 && v_page_stride % per == 0 && v_head_stride % per == 0 &&
        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0) {
        TIS_DISPATCH_DTYPE(dtype, T,
            tis_launch(head_norm_store_vec_kernel<T>, dim3(n), dim3(256), 0, stream, (const T*)qkv, ld, H, G, M, dim, vdim,
                       bias, wq, wk, eps, temp_coef, temp_every, (T*)q_out, ldq, (T*)k_pages, k_page_stride, k_head_stride,
                       (T*)v_pages, v_page_stride, v_head_stride, page_size, num_pages, block_table, bt_stride, positions,
                       row_slot, fault));
        return tis_check_launch("head_norm_store");
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(head_norm_store_kernel<T>, dim3(n), dim3(256), 0, stream, (const T*)qkv, ld, H, G, M, dim, vdim, bias,
                   wq, wk, eps, temp_coef, temp_every, (T*)q_out, ldq, (T*)k_pages, k_page_stride, k_head_stride,
                   (T*)v_pages, v_page_stride, v_head_stride, page_size, num_pages, block_table, bt_stride, positions,
                   row_slot, fault));
    return tis_check_launch("head_norm_store");
}

// ------------------------------------------------------------------------------------------------------------
// Two score maps of a head combined: a row of `a` holds, head by head, the outputs of map 1 and of map 2 (`vdim`
// elements each); out[r, h] = o / sqrt(mean(o^2) + eps) * out_scale with o = a1 - lambda * a2, in 32-bit.  A warp per
// (row, head).
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ a, int lda, float lambda, float eps, float out_scale, T* __restrict__ out,
                    int ldo, const int* __restrict__ row_slot, int n, int H, int vdim) {
    pdl_launch_dependents();
    const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= n * H) return;
    const int r = idx / H, head = idx - r * H;
    if (row_slot != nullptr && row_slot[r] < 0) return;
    pdl_wait();
    const T* a1 = a + (size_t)r * lda + (size_t)head * 2 * vdim;
    const T* a2 = a1 + vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) {
        const float o = fmaf(-lambda, to_f32(a2[j]), to_f32(a1[j]));
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float f = rsqrtf(ss / (float)vdim + eps) * out_scale;
    for (int j = lane; j < vdim; j += 32)
        out[(size_t)r * ldo + (size_t)head * vdim + j] = from_f32<T>(fmaf(-lambda, to_f32(a2[j]), to_f32(a1[j])) * f);
}

TIS_API int tis_diff_combine(int dtype, const void* a, int lda, float lambda, float eps, float out_scale, void* out,
                             int ldo, const int* row_slot, int n, int H, int vdim, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (H <= 0 || vdim <= 0 || lda < 2 * H * vdim || ldo < H * vdim) {
        tis_set_error("diff_combine: %d heads of %d values, row lengths %d in and %d out", H, vdim, lda, ldo);
        return TIS_BAD_SIZE;
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(diff_combine_kernel<T>, dim3((n * H + 3) / 4), dim3(128), 0, stream, (const T*)a, lda, lambda, eps,
                   out_scale, (T*)out, ldo, row_slot, n, H, vdim));
    return tis_check_launch("diff_combine");
}

// ------------------------------------------------------------------------------------------------------------
// Attention of one row and query head over the keys lo..pos of its request's pages, lo = max(0, pos - window + 1)
// (window 0: lo = 0):  score_j = q . k_j * scale - r1[head] * ln(1 + r2[head] * (pos - j)), softmax, times values,
// times sigmoid(gate) element by element (gate_per_head: `gate` holds one number per head, for all its elements).
// r1 null: no bias; gate null: no gate.
// A CTA of 128 threads: 128 keys a tile, a thread a key for the scores; for the values the threads form
// 128 / v_dim groups, each taking every groups-th key of the tile, a thread a value column.
// ------------------------------------------------------------------------------------------------------------
constexpr int WA_THREADS = 128;
constexpr int WA_MAX_COLS = 4;          // value columns a thread keeps: v_dim <= 512

template <typename T>
__global__ void __launch_bounds__(WA_THREADS)
window_attention_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ gate, int ldg, T* __restrict__ out,
                        int ldo, const T* __restrict__ k_pages, size_t k_page_stride, size_t k_head_stride,
                        const T* __restrict__ v_pages, size_t v_page_stride, size_t v_head_stride,
                        const int* __restrict__ block_table, int bt_stride, int num_pages,
                        const int* __restrict__ positions, const int* __restrict__ row_slot, int H, int G, int k_dim,
                        int v_dim, int page_size, int window, float scale, const float* __restrict__ r1,
                        const float* __restrict__ r2, const float* __restrict__ sink, int v_row, int gate_per_head,
                        int* __restrict__ fault) {
    extern __shared__ float smem[];
    __shared__ float red[33];
    __shared__ int page_of[WA_THREADS];
    pdl_launch_dependents();
    const int r = blockIdx.x, head = blockIdx.y;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int kvh = head / (H / G);
    const float b1 = r1 != nullptr ? r1[head] : 0.f, b2 = r1 != nullptr ? r2[head] : 0.f;
    float* qs = smem;                                   // [k_dim]
    float* ps = qs + k_dim;                             // [WA_THREADS]
    float* part = ps + WA_THREADS;                      // [groups][v_dim]
    const int tid = threadIdx.x;
    pdl_wait();
    for (int i = tid; i < k_dim; i += WA_THREADS) qs[i] = to_f32(q[(size_t)r * ldq + (size_t)head * k_dim + i]);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    // value columns
    const int groups = v_dim >= WA_THREADS ? 1 : WA_THREADS / v_dim;
    const int grp = v_dim >= WA_THREADS ? 0 : tid / v_dim;
    const int col0 = v_dim >= WA_THREADS ? tid : tid - grp * v_dim;
    const bool works = grp < groups;
    float acc[WA_MAX_COLS];
#pragma unroll
    for (int a = 0; a < WA_MAX_COLS; ++a) acc[a] = 0.f;
    // a sink is one more term of the denominator, exp(sink[head]), with no value: the running maximum starts there
    float m = sink != nullptr ? sink[head] : -INFINITY, l = sink != nullptr ? 1.f : 0.f;
    __syncthreads();
    for (int base = lo; base < hi; base += WA_THREADS) {
        const int j = base + tid;
        float s = -INFINITY;
        int page = -1;
        if (j < hi) {
            page = block_table[(size_t)slot * bt_stride + j / page_size];
            if (page < 0 || page >= num_pages) {
                atomicExch(fault, 4);
                page = -1;
            } else {
                const T* kr = k_pages + (size_t)page * k_page_stride + (size_t)kvh * k_head_stride +
                              (size_t)(j % page_size) * k_dim;
                float d = 0.f;
                for (int i = 0; i < k_dim; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
                s = d * scale - b1 * logf(1.f + b2 * (float)(pos - j));
            }
        }
        page_of[tid] = page;
        const float m_new = fmaxf(m, block_max(s, red));
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        const float p = (s == -INFINITY || m_new == -INFINITY) ? 0.f : expf(s - m_new);
        l = l * corr + block_sum(p, red);
        m = m_new;
        ps[tid] = p;
#pragma unroll
        for (int a = 0; a < WA_MAX_COLS; ++a) acc[a] *= corr;
        __syncthreads();
        if (works) {
            const int cnt = min(WA_THREADS, hi - base);
            for (int t = grp; t < cnt; t += groups) {
                const int pg = page_of[t];
                if (pg < 0) continue;
                const float pt = ps[t];
                const T* vr = v_pages + (size_t)pg * v_page_stride + (size_t)kvh * v_head_stride +
                              (size_t)((base + t) % page_size) * v_row;
#pragma unroll
                for (int a = 0; a < WA_MAX_COLS; ++a) {
                    const int c = col0 + a * WA_THREADS;
                    if (c < v_dim) acc[a] = fmaf(pt, to_f32(vr[c]), acc[a]);
                }
            }
        }
        __syncthreads();
    }
    if (groups > 1) {
        if (works) part[grp * v_dim + col0] = acc[0];
        __syncthreads();
        if (tid < v_dim) {
            float s = 0.f;
            for (int g2 = 0; g2 < groups; ++g2) s += part[g2 * v_dim + tid];
            acc[0] = s;
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (grp == 0) {
#pragma unroll
        for (int a = 0; a < WA_MAX_COLS; ++a) {
            const int c = col0 + a * WA_THREADS;
            if (c < v_dim) {
                float o = acc[a] * inv;
                if (gate != nullptr) {
                    const float gv = to_f32(gate_per_head ? gate[(size_t)r * ldg + head]
                                                          : gate[(size_t)r * ldg + (size_t)head * v_dim + c]);
                    o = o / (1.f + expf(-gv));
                }
                out[(size_t)r * ldo + (size_t)head * v_dim + c] = from_f32<T>(o);
            }
        }
    }
}

TIS_API int tis_window_attention(int dtype, const void* q, int ldq, const void* gate, int ldg, void* out, int ldo,
                                 const void* k_pages, size_t k_page_stride, size_t k_head_stride, const void* v_pages,
                                 size_t v_page_stride, size_t v_head_stride, const int* block_table, int bt_stride,
                                 int num_pages, const int* positions, const int* row_slot, int n, int H, int G,
                                 int k_dim, int v_dim, int page_size, int window, float scale, const float* r1,
                                 const float* r2, const float* sink, int v_row, int gate_per_head, int* fault,
                                 cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (H <= 0 || G <= 0 || H % G || k_dim <= 0 || v_dim <= 0 || v_dim > WA_THREADS * WA_MAX_COLS || page_size <= 0 ||
        window < 0 || v_row < v_dim) {
        tis_set_error("window_attention: %d query heads, %d kv heads, key width %d, value width %d (at most %d), "
                      "page size %d, window %d", H, G, k_dim, v_dim, WA_THREADS * WA_MAX_COLS, page_size, window);
        return TIS_BAD_SIZE;
    }
    const int groups = v_dim >= WA_THREADS ? 1 : WA_THREADS / v_dim;
    const size_t smem = sizeof(float) * ((size_t)k_dim + WA_THREADS + (size_t)groups * v_dim);
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(window_attention_kernel<T>, dim3(n, H), dim3(WA_THREADS), smem, stream, (const T*)q, ldq,
                   (const T*)gate, ldg, (T*)out, ldo, (const T*)k_pages, k_page_stride, k_head_stride, (const T*)v_pages,
                   v_page_stride, v_head_stride, block_table, bt_stride, num_pages, positions, row_slot, H, G, k_dim,
                   v_dim, page_size, window, scale, r1, r2, sink, v_row, gate_per_head, fault));
    return tis_check_launch("window_attention");
}

// ------------------------------------------------------------------------------------------------------------
// The delta rule with a decay per head and key channel.  Per request and head a state S (k_dim x v_dim, 32-bit):
//   q^ = q / sqrt(sum q^2 + unit_eps) * q_scale,  k^ = k / sqrt(sum k^2 + unit_eps)          (per head)
//   beta = sigmoid(b),  g_i = exp(-exp(A_log[head]) * softplus(a_i + dt_bias_i))               (per key channel i)
//   S <- diag(g) S;  u = beta * (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^
//   out = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate)                                   (over v_dim)
// A row of `qkv` holds the queries and keys of G heads (k_dim each) and the values of H heads (v_dim each).
// One CTA per (head, row); the CTAs of rows that are not the first of their request in the step leave at once (rows
// are the slowest grid dimension, so that the CTAs with work are not queued behind thousands of those).
// Every column of S is a recurrence of its own: a thread keeps one column (in registers when DIM > 0 is the key
// width, else in shared memory, or in place in global memory where it does not fit there; up to 1024 columns).
// Tokens are taken CHUNK at a time: all threads prepare q^, k^, g, beta and v of the chunk, then every thread walks
// its column through the chunk without a barrier, then the outputs of the chunk are normalised, a warp a token.
// ------------------------------------------------------------------------------------------------------------
constexpr int DELTA_CHUNK = 16;

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
// what a gate does to the projection it is made from: 0 sigmoid, 1 silu
__device__ __forceinline__ float gate_f(float x, int act) { const float s = 1.f / (1.f + expf(-x)); return act == 1 ? x * s : s; }
// where the decay of a token comes from: a projection per head and key channel, a projection per head, or a constant
// per head (`A_log` then holds the constants themselves and the recurrence is plain linear attention: q, k and v pass
// silu instead of the unit norms, and the state takes k v^T without the correction towards v)
// or (DECAY_FORGET_GATE) a forget gate per head and key channel that also decides what is written: with `a_in` the
// gate's projection, `dt_bias` its bias and `A_log` a lower bound per head and key channel, f = low + (1 - low) *
// sigmoid(a + bias), S <- diag(f) S + (1 - f) v^T, o = S^T silu(q): the key is 1 - f, there is no key projection (a
// row of `qkv` holds the queries and then the values), no unit norms and no correction towards v
// or (DECAY_LOG_SIGMOID) a gate per head and key channel raised to a power: with `a_in` the gate's projection, `dt_bias`
// its bias and `A_log` the power itself per head (1 / tau), g = sigmoid(a + bias)^power = exp(-power * softplus(-(a + bias))),
// S <- diag(g) S + k v^T, o = S^T (q * q_scale): gated linear attention, no unit norms, no correction
// or (DECAY_STEP) a step size per head and token: with `a_in` (n, H) its projection and `dt_bias` (H) its bias,
// dt = softplus(a + bias), S <- exp(-exp(A_log[head]) * dt) S + k (dt v)^T, o = S^T q: a selective state space in its
// recurrent form (k is the input matrix B, q the output matrix C, v the head's inputs); the outputs leave unnormalised
enum { DECAY_PER_CHANNEL = 0, DECAY_PER_HEAD = 1, DECAY_CONSTANT = 2, DECAY_FORGET_GATE = 3, DECAY_LOG_SIGMOID = 4,
       DECAY_STEP = 5 };

template <typename T, int DIM>
__global__ void __launch_bounds__(DIM > 0 ? 256 : 1024)
delta_rule_kernel(const T* __restrict__ qkv, int ld, const T* __restrict__ b_in, int ldb, const T* __restrict__ a_in,
                  int lda, const T* __restrict__ gate, int ldg, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ norm_w, float eps, float unit_eps,
                  float q_scale, float* __restrict__ state, size_t state_stride, T* __restrict__ out, int ldo,
                  const int* __restrict__ row_slot, const int* __restrict__ row_last, int H, int G, int k_dim_rt,
                  int v_dim, int decay_mode, int gate_act, float* __restrict__ o_raw, int state_in_place) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    const int head = blockIdx.x, r0 = blockIdx.y;
    const int slot = row_slot[r0];
    if (slot < 0) return;
    if (r0 > 0 && row_slot[r0 - 1] == slot) return;
    const int k_dim = DIM > 0 ? DIM : k_dim_rt;
    const int rows = row_last[r0] - r0 + 1;
    const int kvh = head / (H / G);
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    float* qs = smem;                                   // [CHUNK][k_dim]
    float* ks = qs + DELTA_CHUNK * k_dim;
    float* gs = ks + DELTA_CHUNK * k_dim;
    float* vs = gs + DELTA_CHUNK * k_dim;               // [CHUNK][v_dim]
    float* os = vs + DELTA_CHUNK * v_dim;               // [CHUNK][v_dim]
    float* betas = os + DELTA_CHUNK * v_dim;            // [CHUNK]
    float* S_sh = betas + DELTA_CHUNK;                  // [k_dim][v_dim] when DIM == 0
    const bool plain = decay_mode == DECAY_CONSTANT;
    const bool forget = decay_mode == DECAY_FORGET_GATE;
    const bool gated = decay_mode == DECAY_LOG_SIGMOID;
    const bool stepped = decay_mode == DECAY_STEP;
    const bool corrects = !plain && !forget && !gated && !stepped;   // the delta rule proper: the state is corrected towards v
    const float decay_rate = (plain || gated) ? A_log[head] : (forget ? 0.f : expf(A_log[head]));
    float* S_glob = state + (size_t)slot * state_stride + (size_t)head * k_dim * v_dim;
    // a state too large for shared memory is walked where it lies (DIM == 0 only): a thread touches its own column alone
    const bool in_place = DIM == 0 && state_in_place != 0;
    if (in_place) S_sh = S_glob;
    constexpr int REG = DIM > 0 ? DIM : 1;
    float S[REG];
    pdl_wait();
    if (tid < v_dim) {
        if (DIM > 0) {
#pragma unroll
            for (int i = 0; i < REG; ++i) S[i] = S_glob[(size_t)i * v_dim + tid];
        } else if (!in_place) {
            for (int i = 0; i < k_dim; ++i) S_sh[i * v_dim + tid] = S_glob[(size_t)i * v_dim + tid];
        }
    }
    const int q_off = kvh * k_dim, k_off = G * k_dim + kvh * k_dim, v_off = (forget ? 1 : 2) * G * k_dim + head * v_dim;
    for (int c0 = 0; c0 < rows; c0 += DELTA_CHUNK) {
        const int cnt = min(DELTA_CHUNK, rows - c0);
        __syncthreads();                                // the chunk before is done with the shared arrays
        for (int t = warp; t < cnt; t += nwarps) {
            const T* row = qkv + (size_t)(r0 + c0 + t) * ld;
            if (forget) {
                const T* arow = a_in + (size_t)(r0 + c0 + t) * lda + (size_t)head * k_dim;
                for (int i = lane; i < k_dim; i += 32) {
                    const float low = A_log[head * k_dim + i];
                    const float open = 1.f / (1.f + expf(to_f32(arow[i]) + dt_bias[head * k_dim + i]));   // 1 - sigmoid
                    qs[t * k_dim + i] = silu_f(to_f32(row[q_off + i]));
                    ks[t * k_dim + i] = (1.f - low) * open;                      // 1 - f
                    gs[t * k_dim + i] = low + (1.f - low) * (1.f - open);        // f
                }
                for (int j = lane; j < v_dim; j += 32) vs[t * v_dim + j] = to_f32(row[v_off + j]);
                if (lane == 0) betas[t] = 1.f;
                continue;
            }
            if (gated || stepped) {
                const size_t rr = (size_t)(r0 + c0 + t);
                const float dtv = stepped ? softplus_f(to_f32(a_in[rr * lda + head]) + dt_bias[head]) : 1.f;
                const float whole = expf(-decay_rate * dtv);
                for (int i = lane; i < k_dim; i += 32) {
                    qs[t * k_dim + i] = to_f32(row[q_off + i]) * q_scale;
                    ks[t * k_dim + i] = to_f32(row[k_off + i]);
                    gs[t * k_dim + i] = stepped ? whole : expf(-decay_rate * softplus_f(
                        -(to_f32(a_in[rr * lda + (size_t)head * k_dim + i]) + dt_bias[head * k_dim + i])));
                }
                for (int j = lane; j < v_dim; j += 32) vs[t * v_dim + j] = to_f32(row[v_off + j]);
                if (lane == 0) betas[t] = dtv;
                continue;
            }
            float sq = 0.f, sk = 0.f;
            for (int i = lane; i < k_dim; i += 32) {
                const float qv = to_f32(row[q_off + i]), kv = to_f32(row[k_off + i]);
                sq += qv * qv;
                sk += kv * kv;
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.f / sqrtf(sk + unit_eps);
            if (plain) {
                for (int i = lane; i < k_dim; i += 32) {
                    qs[t * k_dim + i] = silu_f(to_f32(row[q_off + i]));
                    ks[t * k_dim + i] = silu_f(to_f32(row[k_off + i]));
                    gs[t * k_dim + i] = decay_rate;
                }
                for (int j = lane; j < v_dim; j += 32) vs[t * v_dim + j] = silu_f(to_f32(row[v_off + j]));
                if (lane == 0) betas[t] = 1.f;
                continue;
            }
            const size_t a_at = decay_mode == DECAY_PER_HEAD ? (size_t)head : (size_t)head * k_dim;
            const int a_step = decay_mode == DECAY_PER_HEAD ? 0 : 1;
            for (int i = lane; i < k_dim; i += 32) {
                qs[t * k_dim + i] = to_f32(row[q_off + i]) * fq;
                ks[t * k_dim + i] = to_f32(row[k_off + i]) * fk;
                const float a = to_f32(a_in[(size_t)(r0 + c0 + t) * lda + a_at + i * a_step]) + dt_bias[a_at + i * a_step];
                gs[t * k_dim + i] = expf(-decay_rate * softplus_f(a));
            }
            for (int j = lane; j < v_dim; j += 32) vs[t * v_dim + j] = to_f32(row[v_off + j]);
            if (lane == 0) {
                const float bv = to_f32(b_in[(size_t)(r0 + c0 + t) * ldb + head]);
                betas[t] = 1.f / (1.f + expf(-bv));
            }
        }
        __syncthreads();
        if (tid < v_dim) {
            for (int t = 0; t < cnt; ++t) {
                const float* kt = ks + t * k_dim;
                const float* qt = qs + t * k_dim;
                const float* gt = gs + t * k_dim;
                float dot = 0.f, o = 0.f;
                if (DIM > 0) {
#pragma unroll
                    for (int i = 0; i < REG; ++i) {
                        S[i] *= gt[i];
                        dot = fmaf(S[i], kt[i], dot);
                    }
                    const float u = corrects ? betas[t] * (vs[t * v_dim + tid] - dot) : betas[t] * vs[t * v_dim + tid];
#pragma unroll
                    for (int i = 0; i < REG; ++i) {
                        S[i] = fmaf(kt[i], u, S[i]);
                        o = fmaf(S[i], qt[i], o);
                    }
                } else {
                    for (int i = 0; i < k_dim; ++i) {
                        const float s = S_sh[i * v_dim + tid] * gt[i];
                        S_sh[i * v_dim + tid] = s;
                        dot = fmaf(s, kt[i], dot);
                    }
                    const float u = corrects ? betas[t] * (vs[t * v_dim + tid] - dot) : betas[t] * vs[t * v_dim + tid];
                    for (int i = 0; i < k_dim; ++i) {
                        const float s = fmaf(kt[i], u, S_sh[i * v_dim + tid]);
                        S_sh[i * v_dim + tid] = s;
                        o = fmaf(s, qt[i], o);
                    }
                }
                os[t * v_dim + tid] = o;
            }
        }
        __syncthreads();
        if (o_raw != nullptr) {                         // the outputs leave as they are, for a norm over whole rows
            for (int idx = tid; idx < cnt * v_dim; idx += nthr) {
                const int t = idx / v_dim, j = idx - t * v_dim;
                o_raw[(size_t)(r0 + c0 + t) * H * v_dim + (size_t)head * v_dim + j] = os[idx];
            }
            continue;
        }
        for (int t = warp; t < cnt; t += nwarps) {
            float ss = 0.f;
            for (int j = lane; j < v_dim; j += 32) { const float o = os[t * v_dim + j]; ss += o * o; }
            ss = warp_sum(ss);
            const float f = rsqrtf(ss / (float)v_dim + eps);
            const size_t rr = (size_t)(r0 + c0 + t);
            for (int j = lane; j < v_dim; j += 32) {
                float o = os[t * v_dim + j] * f * norm_w[j];
                if (gate != nullptr) o *= gate_f(to_f32(gate[rr * ldg + head * v_dim + j]), gate_act);
                out[rr * ldo + head * v_dim + j] = from_f32<T>(o);
            }
        }
    }
    if (tid < v_dim) {
        if (DIM > 0) {
#pragma unroll
            for (int i = 0; i < REG; ++i) S_glob[(size_t)i * v_dim + tid] = S[i];
        } else if (!in_place) {
            for (int i = 0; i < k_dim; ++i) S_glob[(size_t)i * v_dim + tid] = S_sh[i * v_dim + tid];
        }
    }
}

// The same recurrence with more parallelism, for key widths LANES * DL and value widths that are multiples of the
// columns a CTA takes: LANES lanes share a column of one head's state (lane p keeps the key channels p * DL .. + DL - 1
// of it in registers) and add their partial sums with shuffles; a CTA takes COLS columns: 32 with four lanes each, or,
// with eight lanes each, 64 (sixteen warps: a scheduler has four recurrences to switch between) or 16 (four times the
// CTAs, for steps of few requests, where a head's columns are all the parallelism there is), or, with sixteen lanes
// each, 8 (a prompt of one request: a thread's share of a token's work is halved again and twice the warps walk).  The
// chunk's q^, k^ and g lie in shared memory with four floats of padding after every lane's share, so that the lanes of
// a column read different banks with 16-byte loads.  A chunk is prepared by all threads, NT / 16 to a token; the raw
// values of the next chunk are loaded into registers before the current chunk is walked.  The outputs leave
// unnormalised, in 32-bit (`o_raw`, (n, H * v_dim)); delta_out_norm_kernel normalises them.
// MODE 0: the delta rule (decays from projections, the state corrected towards v); 1: a constant decay per head,
// silu on q, k and v, no correction; 2: the forget gate of DECAY_FORGET_GATE; 3: the powered gate of DECAY_LOG_SIGMOID;
// 4: the step size of DECAY_STEP.
template <typename T, int DL, int LANES, int COLS, int MODE>
__global__ void __launch_bounds__(COLS * LANES)
delta_rule_split_kernel(const T* __restrict__ qkv, int ld, const T* __restrict__ b_in, int ldb, const T* __restrict__ a_in,
                        int lda, const float* __restrict__ A_log, const float* __restrict__ dt_bias, float unit_eps,
                        float q_scale, float* __restrict__ state, size_t state_stride, float* __restrict__ o_raw,
                        const int* __restrict__ row_slot, const int* __restrict__ row_last,
                        const int* __restrict__ seg_row0, int H, int G, int v_dim, int decay_mode) {
    constexpr int KDIM = LANES * DL, QP = DL + 4, ROW = LANES * QP, NT = COLS * LANES;
    constexpr int PT = NT / DELTA_CHUNK;                // threads that prepare a token
    constexpr int CH = KDIM / PT, VPT = COLS / PT;      // key channels and value columns of each
    static_assert(KDIM % PT == 0 && COLS % PT == 0 && DL % 2 == 0, "widths");
    __shared__ __align__(16) float qs[DELTA_CHUNK][ROW];
    __shared__ __align__(16) float ks[DELTA_CHUNK][ROW];
    __shared__ __align__(16) float gs[DELTA_CHUNK][ROW];
    __shared__ float vs[DELTA_CHUNK][COLS];
    __shared__ float betas[DELTA_CHUNK];
    pdl_launch_dependents();
    const int head = blockIdx.x, col0 = blockIdx.y * COLS;
    // grid.z: the requests of the step, by their first rows (`seg_row0`), or, without that list, every row (the CTAs
    // of rows that are not the first of their request leave at once)
    const int r0 = seg_row0 != nullptr ? seg_row0[blockIdx.z] : (int)blockIdx.z;
    const int slot = row_slot[r0];
    if (slot < 0) return;
    if (r0 > 0 && row_slot[r0 - 1] == slot) return;
    const int rows = row_last[r0] - r0 + 1;
    const int kvh = head / (H / G);
    const int tid = threadIdx.x;
    const int col = tid / LANES, part = tid % LANES;
    // PLAIN: the decay is a constant per head and the state takes k v^T as it is, so the walk needs neither the decays of
    // the chunk nor the first of its two sums over the lanes of a column
    constexpr bool plain = MODE == 1, forget = MODE == 2, gated = MODE == 3, stepped = MODE == 4;
    const float decay_rate = (plain || gated) ? A_log[head] : (forget ? 0.f : expf(A_log[head]));
    float* S_glob = state + (size_t)slot * state_stride + (size_t)head * KDIM * v_dim + col0 + col;
    float S[DL];
    pdl_wait();
#pragma unroll
    for (int i = 0; i < DL; ++i) S[i] = S_glob[(size_t)(part * DL + i) * v_dim];
    const int q_off = kvh * KDIM, k_off = G * KDIM + kvh * KDIM, v_off = (forget ? 1 : 2) * G * KDIM + head * v_dim + col0;
    const int nv = H * v_dim;
    const int pt = tid / PT, sub = tid % PT;
    const bool per_head = decay_mode == DECAY_PER_HEAD || decay_mode == DECAY_STEP;
    const size_t a_at = per_head ? (size_t)head : (size_t)head * KDIM;
    const int a_step = per_head ? 0 : 1;
    float rq[CH], rk[CH], ra[CH], rv[VPT], rb = 0.f;
    auto fetch = [&](int c0) {
        const bool live = c0 + pt < rows;
        const size_t rr = (size_t)(r0 + c0 + pt);
        const T* row = qkv + rr * ld;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            rq[i] = live ? to_f32(row[q_off + sub * CH + i]) : 0.f;
            rk[i] = (live && !forget) ? to_f32(row[k_off + sub * CH + i]) : 0.f;
            ra[i] = (live && !plain) ? to_f32(a_in[rr * lda + a_at + (sub * CH + i) * a_step]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) rv[i] = live ? to_f32(row[v_off + sub * VPT + i]) : 0.f;
        rb = (live && sub == 0 && MODE == 0) ? to_f32(b_in[rr * ldb + head]) : 0.f;
    };
    float bias[CH], low[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        bias[i] = plain ? 0.f : dt_bias[a_at + (sub * CH + i) * a_step];
        low[i] = forget ? A_log[a_at + sub * CH + i] : 0.f;
    }
    fetch(0);
    for (int c0 = 0; c0 < rows; c0 += DELTA_CHUNK) {
        const int cnt = min(DELTA_CHUNK, rows - c0);
        __syncthreads();                                // the chunk before is done with the shared arrays
        {
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int i = 0; i < CH; ++i) { sq = fmaf(rq[i], rq[i], sq); sk = fmaf(rk[i], rk[i], sk); }
#pragma unroll
            for (int o = 1; o < PT; o <<= 1) {
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
            }
            const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.f / sqrtf(sk + unit_eps);
            // a decay per head is one number for all of a token's key channels: made once, not once a channel
            const float g_head = (a_step == 0 && !plain && !forget && !gated) ? expf(-decay_rate * softplus_f(ra[0] + bias[0])) : 0.f;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int ch = sub * CH + i;
                const int at = ch + (ch / DL) * 4;
                if (forget) {
                    const float open = 1.f / (1.f + expf(ra[i] + bias[i]));     // 1 - sigmoid of the gate
                    qs[pt][at] = silu_f(rq[i]);
                    ks[pt][at] = (1.f - low[i]) * open;                          // 1 - f
                    gs[pt][at] = low[i] + (1.f - low[i]) * (1.f - open);         // f
                } else if (gated || stepped) {
                    qs[pt][at] = rq[i] * q_scale;
                    ks[pt][at] = rk[i];
                    gs[pt][at] = gated ? expf(-decay_rate * softplus_f(-(ra[i] + bias[i]))) : g_head;
                } else {
                    qs[pt][at] = plain ? silu_f(rq[i]) : rq[i] * fq;
                    ks[pt][at] = plain ? silu_f(rk[i]) : rk[i] * fk;
                    gs[pt][at] = plain ? decay_rate : (a_step == 0 ? g_head : expf(-decay_rate * softplus_f(ra[i] + bias[i])));
                }
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) vs[pt][sub * VPT + i] = plain ? silu_f(rv[i]) : rv[i];
            if (sub == 0) betas[pt] = stepped ? softplus_f(ra[0] + bias[0]) : 1.f / (1.f + expf(-rb));
        }
        __syncthreads();
        if (c0 + DELTA_CHUNK < rows) fetch(c0 + DELTA_CHUNK);
        // With registers to spare (the narrow CTAs) a token's vectors are read from shared memory while the token
        // before is walked, so that the recurrence never waits for them.
        constexpr bool AHEAD = NT <= 128 && LANES >= 8;
        float2 kn[AHEAD ? DL / 2 : 1], qn[AHEAD ? DL / 2 : 1], gn[AHEAD ? DL / 2 : 1];
        float vn = 0.f, bn = 0.f;
        auto ahead = [&](int t) {
            if (AHEAD) {
                const float2* kt = reinterpret_cast<const float2*>(&ks[t][part * QP]);
                const float2* qt = reinterpret_cast<const float2*>(&qs[t][part * QP]);
                const float2* gt = reinterpret_cast<const float2*>(&gs[t][part * QP]);
#pragma unroll
                for (int i = 0; i < DL / 2; ++i) { kn[i] = kt[i]; qn[i] = qt[i]; gn[i] = gt[i]; }
                vn = vs[t][col];
                bn = betas[t];
            }
        };
        ahead(0);
        for (int t = 0; t < cnt; ++t) {
            float2 kc[DL / 2], qc[DL / 2], gc[DL / 2];
            float vc, bc;
            if (AHEAD) {
#pragma unroll
                for (int i = 0; i < DL / 2; ++i) { kc[i] = kn[i]; qc[i] = qn[i]; gc[i] = gn[i]; }
                vc = vn;
                bc = bn;
                if (t + 1 < cnt) ahead(t + 1);
            } else {
                const float2* kt = reinterpret_cast<const float2*>(&ks[t][part * QP]);
                const float2* qt = reinterpret_cast<const float2*>(&qs[t][part * QP]);
                const float2* gt = reinterpret_cast<const float2*>(&gs[t][part * QP]);
#pragma unroll
                for (int i = 0; i < DL / 2; ++i) { kc[i] = kt[i]; qc[i] = qt[i]; gc[i] = gt[i]; }
                vc = vs[t][col];
                bc = betas[t];
            }
            float d0 = 0.f, d1 = 0.f, u = vc;
            if (plain) {
#pragma unroll
                for (int i = 0; i < DL; ++i) S[i] *= decay_rate;
            } else if (forget || gated || stepped) {
#pragma unroll
                for (int i = 0; i < DL / 2; ++i) { S[2 * i] *= gc[i].x; S[2 * i + 1] *= gc[i].y; }
                if (stepped) u = bc * vc;
            } else {
#pragma unroll
                for (int i = 0; i < DL / 2; ++i) {
                    S[2 * i] *= gc[i].x; S[2 * i + 1] *= gc[i].y;
                    d0 = fmaf(S[2 * i], kc[i].x, d0); d1 = fmaf(S[2 * i + 1], kc[i].y, d1);
                }
                float dot = d0 + d1;
#pragma unroll
                for (int o = 1; o < LANES; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                u = bc * (vc - dot);
            }
            d0 = d1 = 0.f;
#pragma unroll
            for (int i = 0; i < DL / 2; ++i) {
                S[2 * i] = fmaf(kc[i].x, u, S[2 * i]); S[2 * i + 1] = fmaf(kc[i].y, u, S[2 * i + 1]);
                d0 = fmaf(S[2 * i], qc[i].x, d0); d1 = fmaf(S[2 * i + 1], qc[i].y, d1);
            }
            float o = d0 + d1;
#pragma unroll
            for (int sh = 1; sh < LANES; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
            if (part == 0) o_raw[(size_t)(r0 + c0 + t) * nv + head * v_dim + col0 + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < DL; ++i) S_glob[(size_t)(part * DL + i) * v_dim] = S[i];
}

// out[r, head, :] = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate) for every (row, head): a warp each.
template <typename T>
__global__ void __launch_bounds__(128)
delta_out_norm_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate, int ldg, const float* __restrict__ norm_w,
                      float eps, T* __restrict__ out, int ldo, const int* __restrict__ row_slot, int n, int H, int v_dim,
                      int gate_act) {
    pdl_launch_dependents();
    const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= n * H) return;
    const int r = idx / H, head = idx - r * H;
    if (row_slot[r] < 0) return;
    pdl_wait();
    const float* o = o_raw + (size_t)r * H * v_dim + (size_t)head * v_dim;
    float ss = 0.f;
    for (int j = lane; j < v_dim; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    const float f = rsqrtf(ss / (float)v_dim + eps);
    for (int j = lane; j < v_dim; j += 32) {
        float x = o[j] * f * norm_w[j];
        if (gate != nullptr) x *= gate_f(to_f32(gate[(size_t)r * ldg + head * v_dim + j]), gate_act);
        out[(size_t)r * ldo + head * v_dim + j] = from_f32<T>(x);
    }
}

// out[r, :] = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate) over the whole row (`width` elements, all heads
// together): a CTA a row.
template <typename T>
__global__ void __launch_bounds__(256)
row_out_norm_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate, int ldg, const float* __restrict__ norm_w,
                    float eps, T* __restrict__ out, int ldo, const int* __restrict__ row_slot, int width) {
    __shared__ float red[33];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    if (row_slot[r] < 0) return;
    pdl_wait();
    const float* o = o_raw + (size_t)r * width;
    float ss = 0.f;
    const bool vec = width % 4 == 0 && ((uintptr_t)o_raw | (uintptr_t)norm_w) % 16 == 0;
    if (vec) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(o + j);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) ss = fmaf(o[j], o[j], ss);
    }
    ss = block_sum(ss, red);
    const float f = rsqrtf(ss / (float)width + eps);
    if (vec) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(o + j);
            const float4 w = *reinterpret_cast<const float4*>(norm_w + j);
            float x[4] = {v.x * f * w.x, v.y * f * w.y, v.z * f * w.z, v.w * f * w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (gate != nullptr) x[e] *= gate_f(to_f32(gate[(size_t)r * ldg + j + e]), 0);
                out[(size_t)r * ldo + j + e] = from_f32<T>(x[e]);
            }
        }
        return;
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float x = o[j] * f * norm_w[j];
        if (gate != nullptr) x *= gate_f(to_f32(gate[(size_t)r * ldg + j]), 0);
        out[(size_t)r * ldo + j] = from_f32<T>(x);
    }
}

template <typename T, int DL, int LANES, int COLS>
static int launch_delta_rule_split(const T* qkv, int ld, const T* b_in, int ldb, const T* a_in, int lda, const T* gate, int ldg,
                                   const float* A_log, const float* dt_bias, const float* norm_w, float eps, float unit_eps,
                                   float q_scale, float* state, size_t state_stride, T* out, int ldo, float* o_raw,
                                   const int* row_slot, const int* row_last, const int* seg_row0, int segments, int n,
                                   int H, int G, int v_dim, int decay_mode, int gate_act, cudaStream_t stream) {
    const dim3 grid(H, v_dim / COLS, seg_row0 != nullptr ? segments : n);
    if (decay_mode == DECAY_CONSTANT)
        tis_launch(delta_rule_split_kernel<T, DL, LANES, COLS, 1>, grid, dim3(COLS * LANES), 0, stream, qkv, ld, b_in, ldb, a_in,
                   lda, A_log, dt_bias, unit_eps, q_scale, state, state_stride, o_raw, row_slot, row_last, seg_row0, H, G, v_dim,
                   decay_mode);
    else if (decay_mode == DECAY_FORGET_GATE)
        tis_launch(delta_rule_split_kernel<T, DL, LANES, COLS, 2>, grid, dim3(COLS * LANES), 0, stream, qkv, ld, b_in, ldb, a_in,
                   lda, A_log, dt_bias, unit_eps, q_scale, state, state_stride, o_raw, row_slot, row_last, seg_row0, H, G, v_dim,
                   decay_mode);
    else if (decay_mode == DECAY_LOG_SIGMOID)
        tis_launch(delta_rule_split_kernel<T, DL, LANES, COLS, 3>, grid, dim3(COLS * LANES), 0, stream, qkv, ld, b_in, ldb, a_in,
                   lda, A_log, dt_bias, unit_eps, q_scale, state, state_stride, o_raw, row_slot, row_last, seg_row0, H, G, v_dim,
                   decay_mode);
    else if (decay_mode == DECAY_STEP)
        tis_launch(delta_rule_split_kernel<T, DL, LANES, COLS, 4>, grid, dim3(COLS * LANES), 0, stream, qkv, ld, b_in, ldb, a_in,
                   lda, A_log, dt_bias, unit_eps, q_scale, state, state_stride, o_raw, row_slot, row_last, seg_row0, H, G, v_dim,
                   decay_mode);
    else
        tis_launch(delta_rule_split_kernel<T, DL, LANES, COLS, 0>, grid, dim3(COLS * LANES), 0, stream, qkv, ld, b_in, ldb, a_in,
                   lda, A_log, dt_bias, unit_eps, q_scale, state, state_stride, o_raw, row_slot, row_last, seg_row0, H, G, v_dim,
                   decay_mode);
    int st = tis_check_launch("delta_rule");
    if (st != TIS_OK || decay_mode == DECAY_STEP) return st;      // DECAY_STEP: the caller gates and normalises `o_raw`
    if (decay_mode == DECAY_CONSTANT) {
        tis_launch(row_out_norm_kernel<T>, dim3(n), dim3(256), 0, stream, (const float*)o_raw, gate, ldg, norm_w, eps, out, ldo,
                   row_slot, H * v_dim);
        return tis_check_launch("row_out_norm");
    }
    tis_launch(delta_out_norm_kernel<T>, dim3((n * H + 3) / 4), dim3(128), 0, stream, (const float*)o_raw, gate, ldg, norm_w, eps,
               out, ldo, row_slot, n, H, v_dim, gate_act);
    return tis_check_launch("delta_out_norm");
}

template <typename T, int DIM>
static int launch_delta_rule(const T* qkv, int ld, const T* b_in, int ldb, const T* a_in, int lda, const T* gate, int ldg,
                             const float* A_log, const float* dt_bias, const float* norm_w, float eps, float unit_eps,
                             float q_scale, float* state, size_t state_stride, T* out, int ldo, const int* row_slot,
                             const int* row_last, int n, int H, int G, int k_dim, int v_dim, int decay_mode, int gate_act,
                             float* o_raw, cudaStream_t stream) {
    int threads = (v_dim + 31) / 32 * 32;
    if (threads < 128) threads = 128;                  // warps to prepare and normalise a chunk with
    size_t smem = sizeof(float) * ((size_t)DELTA_CHUNK * (3 * k_dim + 2 * v_dim + 1) + (DIM > 0 ? 0 : (size_t)k_dim * v_dim));
    int in_place = 0;
    if (smem > 200 * 1024) {                           // the state stays in global memory
        in_place = 1;
        smem = sizeof(float) * ((size_t)DELTA_CHUNK * (3 * k_dim + 2 * v_dim + 1));
    }
    if (smem > 200 * 1024 || (in_place && DIM > 0)) {
        tis_set_error("delta_rule: key width %d x value width %d does not fit shared memory", k_dim, v_dim);
        return TIS_BAD_SIZE;
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(delta_rule_kernel<T, DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    tis_launch(delta_rule_kernel<T, DIM>, dim3(H, n), dim3(threads), smem, stream, qkv, ld, b_in, ldb, a_in, lda, gate, ldg,
               A_log, dt_bias, norm_w, eps, unit_eps, q_scale, state, state_stride, out, ldo, row_slot, row_last, H, G,
               k_dim, v_dim, decay_mode, gate_act,
               (decay_mode == DECAY_CONSTANT || decay_mode == DECAY_STEP) ? o_raw : (float*)nullptr, in_place);
    int st = tis_check_launch("delta_rule");
    if (st != TIS_OK || decay_mode != DECAY_CONSTANT) return st;
    tis_launch(row_out_norm_kernel<T>, dim3(n), dim3(256), 0, stream, (const float*)o_raw, gate, ldg, norm_w, eps, out, ldo,
               row_slot, H * v_dim);
    return tis_check_launch("row_out_norm");
}

// Whether tis_delta_rule takes the kernel that splits a head's columns over CTAs for these widths (it then needs
// `o_raw`, n * H * v_dim floats of scratch).
TIS_API int tis_delta_rule_splits(int k_dim, int v_dim) {
    if (v_dim % 32) return 0;
    switch (k_dim) { case 16: case 32: case 48: case 64: case 96: case 128: return 1; default: return 0; }
}

static int matrix_state_recurrence(int dtype, const void* qkv, int ld, const void* b_in, int ldb, const void* a_in, int lda,
                                   const void* gate, int ldg, const float* A_log, const float* dt_bias, const float* norm_w,
                                   float eps, float unit_eps, float q_scale, float* state, size_t state_stride, void* out,
                                   int ldo, float* o_raw, const int* row_slot, const int* row_last, int n, int H, int G,
                                   int k_dim, int v_dim, int narrow, const int* seg_row0, int segments, int decay_mode,
                                   int gate_act, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (decay_mode < DECAY_PER_CHANNEL || decay_mode > DECAY_STEP || gate_act < 0 || gate_act > 1 ||
        ((decay_mode == DECAY_CONSTANT || decay_mode == DECAY_STEP) && o_raw == nullptr)) {
        tis_set_error("delta_rule: decay mode %d, gate activation %d%s", decay_mode, gate_act,
                      o_raw == nullptr ? ", no scratch for the outputs" : "");
        return TIS_BAD_SIZE;
    }
    if (n > 65535) {
        tis_set_error("delta_rule: %d rows in one step (at most 65535)", n);
        return TIS_BAD_SIZE;
    }
    if (o_raw != nullptr && H > 0 && G > 0 && H % G == 0 && tis_delta_rule_splits(k_dim, v_dim)) {
#define TIS_DELTA_SPLIT(K, DL, LANES, COLS)                                                                           \
    if (k_dim == K)                                                                                                    \
        TIS_DISPATCH_DTYPE(dtype, T, return (launch_delta_rule_split<T, DL, LANES, COLS>((const T*)qkv, ld,            \
            (const T*)b_in, ldb, (const T*)a_in, lda, (const T*)gate, ldg, A_log, dt_bias, norm_w, eps, unit_eps,      \
            q_scale, state, state_stride, (T*)out, ldo, o_raw, row_slot, row_last, seg_row0, segments, n, H, G, v_dim,       \
            decay_mode, gate_act, stream)));
        if (v_dim % 8 == 0 && narrow >= 2) {            // sixteen lanes a column, 8 columns a CTA: one or two requests
            TIS_DELTA_SPLIT(32, 2, 16, 8)
            TIS_DELTA_SPLIT(64, 4, 16, 8)
            TIS_DELTA_SPLIT(128, 8, 16, 8)
        }
        if (v_dim % 64 == 0 && !narrow) {               // eight lanes a column, 64 columns a CTA
            TIS_DELTA_SPLIT(32, 4, 8, 64)
            TIS_DELTA_SPLIT(64, 8, 8, 64)
            TIS_DELTA_SPLIT(96, 12, 8, 64)
            TIS_DELTA_SPLIT(128, 16, 8, 64)
        }
        if (v_dim % 16 == 0 && narrow) {                // eight lanes a column, 16 columns a CTA
            TIS_DELTA_SPLIT(32, 4, 8, 16)
            TIS_DELTA_SPLIT(64, 8, 8, 16)
            TIS_DELTA_SPLIT(96, 12, 8, 16)
            TIS_DELTA_SPLIT(128, 16, 8, 16)
        }
        TIS_DELTA_SPLIT(16, 4, 4, 32)
        TIS_DELTA_SPLIT(32, 8, 4, 32)
        TIS_DELTA_SPLIT(48, 12, 4, 32)
        TIS_DELTA_SPLIT(64, 16, 4, 32)
        TIS_DELTA_SPLIT(96, 24, 4, 32)
        TIS_DELTA_SPLIT(128, 32, 4, 32)
#undef TIS_DELTA_SPLIT
    }
    if (H <= 0 || G <= 0 || H % G || k_dim <= 0 || v_dim <= 0 || v_dim > 1024) {
        tis_set_error("delta_rule: %d heads, %d query/key heads, key width %d, value width %d (at most 1024)", H, G, k_dim,
                      v_dim);
        return TIS_BAD_SIZE;
    }
#define TIS_DELTA_CASE(D)                                                                                              \
    case D:                                                                                                            \
        TIS_DISPATCH_DTYPE(dtype, T, return launch_delta_rule<T, D>((const T*)qkv, ld, (const T*)b_in, ldb,            \
            (const T*)a_in, lda, (const T*)gate, ldg, A_log, dt_bias, norm_w, eps, unit_eps, q_scale, state,           \
            state_stride, (T*)out, ldo, row_slot, row_last, n, H, G, k_dim, v_dim, decay_mode, gate_act, o_raw,        \
            stream));                                                                                                 \
        break;
    switch (v_dim <= 256 ? k_dim : 0) {                 // a column's state in registers: CTAs of up to 256 columns
        TIS_DELTA_CASE(16)
        TIS_DELTA_CASE(32)
        TIS_DELTA_CASE(64)
        TIS_DELTA_CASE(128)
        default: break;
    }
#undef TIS_DELTA_CASE
    TIS_DISPATCH_DTYPE(dtype, T, return launch_delta_rule<T, 0>((const T*)qkv, ld, (const T*)b_in, ldb, (const T*)a_in,
        lda, (const T*)gate, ldg, A_log, dt_bias, norm_w, eps, unit_eps, q_scale, state, state_stride, (T*)out, ldo,
        row_slot, row_last, n, H, G, k_dim, v_dim, decay_mode, gate_act, o_raw, stream));
    return TIS_OK;
}

// The delta rule.  decay_per_head 0: `a_in` (n, H * k_dim) and `dt_bias` (H * k_dim), a decay per head and key channel;
// 1: `a_in` (n, H) and `dt_bias` (H), one per head.  gate_act: 0 sigmoid, 1 silu.
TIS_API int tis_delta_rule(int dtype, const void* qkv, int ld, const void* b_in, int ldb, const void* a_in, int lda,
                           const void* gate, int ldg, const float* A_log, const float* dt_bias, const float* norm_w,
                           float eps, float unit_eps, float q_scale, float* state, size_t state_stride, void* out,
                           int ldo, float* o_raw, const int* row_slot, const int* row_last, int n, int H, int G,
                           int k_dim, int v_dim, int narrow, const int* seg_row0, int segments, int decay_per_head,
                           int gate_act, cudaStream_t stream) {
    return matrix_state_recurrence(dtype, qkv, ld, b_in, ldb, a_in, lda, gate, ldg, A_log, dt_bias, norm_w, eps, unit_eps,
                                   q_scale, state, state_stride, out, ldo, o_raw, row_slot, row_last, n, H, G, k_dim, v_dim,
                                   narrow, seg_row0, segments, decay_per_head ? DECAY_PER_HEAD : DECAY_PER_CHANNEL, gate_act,
                                   stream);
}

// Linear attention with a constant decay per head (`decay`, H numbers): S <- decay S + silu(k) silu(v)^T, o = S^T silu(q);
// the outputs of a row's heads together are divided by their root mean square, multiplied by `norm_w` (H * v_dim) and by
// sigmoid(gate).  `o_raw`: n * H * v_dim floats of scratch.  The recurrence is walked by the delta rule's kernels.
TIS_API int tis_linear_attention(int dtype, const void* qkv, int ld, const void* gate, int ldg, const float* decay,
                                 const float* norm_w, float eps, float* state, size_t state_stride, void* out, int ldo,
                                 float* o_raw, const int* row_slot, const int* row_last, int n, int H, int k_dim, int v_dim,
                                 int narrow, const int* seg_row0, int segments, cudaStream_t stream) {
    return matrix_state_recurrence(dtype, qkv, ld, nullptr, 0, nullptr, 0, gate, ldg, decay, nullptr, norm_w, eps, 0.f, 1.f,
                                   state, state_stride, out, ldo, o_raw, row_slot, row_last, n, H, H, k_dim, v_dim, narrow,
                                   seg_row0, segments, DECAY_CONSTANT, 0, stream);
}

// The recurrence with a forget gate per head and key channel (DECAY_FORGET_GATE): a row of `qv` holds the queries of H
// heads (k_dim each, before silu) and the values of H heads (v_dim each); `f_in` (n, H * k_dim) the gate's projection,
// `f_bias` its bias, `lower` the gate's lower bounds (H * k_dim each).  Per head out = o / sqrt(mean(o^2) + eps) * norm_w
// (v_dim weights, the same for every head).  `o_raw`: n * H * v_dim floats of scratch where tis_delta_rule_splits.
TIS_API int tis_forget_gate_recurrence(int dtype, const void* qv, int ld, const void* f_in, int ldf, const float* lower,
                                       const float* f_bias, const float* norm_w, float eps, float* state,
                                       size_t state_stride, void* out, int ldo, float* o_raw, const int* row_slot,
                                       const int* row_last, int n, int H, int k_dim, int v_dim, int narrow,
                                       const int* seg_row0, int segments, cudaStream_t stream) {
    return matrix_state_recurrence(dtype, qv, ld, nullptr, 0, f_in, ldf, nullptr, 0, lower, f_bias, norm_w, eps, 0.f, 1.f,
                                   state, state_stride, out, ldo, o_raw, row_slot, row_last, n, H, H, k_dim, v_dim, narrow,
                                   seg_row0, segments, DECAY_FORGET_GATE, 0, stream);
}

// Gated linear attention (DECAY_LOG_SIGMOID): a row of `qkv` holds the queries and keys of H heads (k_dim each) and the
// values of H heads (v_dim each); `a_in` (n, H * k_dim) the gate's projection, `a_bias` (H * k_dim) its bias, `power` (H)
// the exponent of the gate.  alpha = sigmoid(a + bias)^power; S <- diag(alpha) S + k v^T; o = S^T (q * q_scale); per head
// out = o / sqrt(mean(o^2) + eps) * norm_w (v_dim weights, the same for every head) * act(gate).  `o_raw`: n * H * v_dim
// floats of scratch where tis_delta_rule_splits.
TIS_API int tis_gated_linear_attention(int dtype, const void* qkv, int ld, const void* a_in, int lda, const float* power,
                                       const float* a_bias, const void* gate, int ldg, const float* norm_w, float eps,
                                       float q_scale, float* state, size_t state_stride, void* out, int ldo, float* o_raw,
                                       const int* row_slot, const int* row_last, int n, int H, int k_dim, int v_dim,
                                       int narrow, const int* seg_row0, int segments, int gate_act, cudaStream_t stream) {
    return matrix_state_recurrence(dtype, qkv, ld, nullptr, 0, a_in, lda, gate, ldg, power, a_bias, norm_w, eps, 0.f, q_scale,
                                   state, state_stride, out, ldo, o_raw, row_slot, row_last, n, H, H, k_dim, v_dim, narrow,
                                   seg_row0, segments, DECAY_LOG_SIGMOID, gate_act, stream);
}

// A selective state space in its recurrent form (DECAY_STEP): a row of `cbx` holds the output matrices C and then the input
// matrices B of G groups (`state_dim` each) and then the inputs x of H heads (v_dim each); `dt_in` (n, H) the step's
// projection, `dt_bias`, `A_log` (H).  dt = softplus(dt_in + dt_bias); S <- exp(-exp(A_log) dt) S + B (dt x)^T;
// o_raw = S^T C, 32-bit, (n, H * v_dim): what follows (a skip, a gate, a norm) is the caller's.
TIS_API int tis_state_space_scan(int dtype, const void* cbx, int ld, const void* dt_in, int ldd, const float* A_log,
                                 const float* dt_bias, float* state, size_t state_stride, float* o_raw, const int* row_slot,
                                 const int* row_last, int n, int H, int G, int state_dim, int v_dim, int narrow,
                                 const int* seg_row0, int segments, cudaStream_t stream) {
    return matrix_state_recurrence(dtype, cbx, ld, nullptr, 0, dt_in, ldd, nullptr, 0, A_log, dt_bias, nullptr, 0.f, 0.f, 1.f,
                                   state, state_stride, nullptr, 0, o_raw, row_slot, row_last, n, H, G, state_dim, v_dim,
                                   narrow, seg_row0, segments, DECAY_STEP, 0, stream);
}
