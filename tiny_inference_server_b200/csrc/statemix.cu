// Row-wise kernels around mixers that keep state:
//   * an embedding with a second, hashed table addressed by the pair (previous token, token), the previous token of a
//     request being part of its state;
//   * an RMS norm in groups (every one of `groups` equal consecutive parts of a row by its own root mean square) that
//     first adds up to two pending updates to the 32-bit residual stream and writes up to two outputs with weights of
//     their own: what a layer whose two sublayers read the same stream needs in one pass;
//   * the step between the projections and the cache of an attention whose values are its keys before rotation:
//     rotate queries in place, write rotated keys as key rows and the unrotated keys as value rows;
//   * what follows the scan of a selective state space: skip, gate, norm in groups.
//
// One CTA per row of the step.  A row whose request slot is negative is padding.
#include "common.cuh"

namespace {

constexpr int FEW_GROUPS = 8;

// out = row * rsqrt(mean over the part + eps) * w, part by part; `row` (d floats) lies in shared memory and is complete
// (the caller has synchronised).  Up to FEW_GROUPS parts: every thread sums its share of every part in registers, one
// reduction over the CTA gives all the parts' sums at once (in a fixed order: the same bits every time), and the outputs
// leave in 16-byte vectors where the sizes allow; more parts: a warp a part.  `red`: FEW_GROUPS * 33 floats.
template <typename O>
__device__ __forceinline__ void grouped_norm_write(const float* row, int d, int groups, float eps, const float* __restrict__ w1,
                                                   O* __restrict__ out1, const float* __restrict__ w2, O* __restrict__ out2,
                                                   float* __restrict__ back, float* red) {
    const int per = d / groups;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    if (groups > FEW_GROUPS) {
        for (int g = warp; g < groups; g += nw) {
            const float* part = row + (size_t)g * per;
            float ss = 0.f;
            for (int i = lane; i < per; i += 32) ss = fmaf(part[i], part[i], ss);
            ss = warp_sum(ss);
            const float f = rsqrtf(ss / (float)per + eps);
            for (int i = lane; i < per; i += 32) {
                const int c = g * per + i;
                const float v = part[i] * f;
                if (back != nullptr) back[c] = v * w1[c];
                else if (out1 != nullptr) out1[c] = from_f32<O>(v * w1[c]);
                if (out2 != nullptr) out2[c] = from_f32<O>(v * w2[c]);
            }
        }
        return;
    }
    float part[FEW_GROUPS];
#pragma unroll
    for (int k = 0; k < FEW_GROUPS; ++k) part[k] = 0.f;
    for (int i = tid; i < d; i += blockDim.x) {
        const float v = row[i];
        const int g = i / per;
#pragma unroll
        for (int k = 0; k < FEW_GROUPS; ++k) part[k] = (k == g) ? fmaf(v, v, part[k]) : part[k];
    }
#pragma unroll
    for (int k = 0; k < FEW_GROUPS; ++k) {
        if (k < groups) {
            const float v = warp_sum(part[k]);
            if (lane == 0) red[k * 33 + warp] = v;
        }
    }
    __syncthreads();
    if (tid < groups) {
        float t = 0.f;
        for (int w = 0; w < nw; ++w) t += red[tid * 33 + w];
        red[tid * 33 + 32] = rsqrtf(t / (float)per + eps);
    }
    __syncthreads();
    constexpr int N = Vec16<O>::N;
    const bool vec = per % N == 0 && back == nullptr &&
                     (((uintptr_t)out1 | (uintptr_t)out2 | (uintptr_t)w1 | (uintptr_t)w2) % 16) == 0;
    if (vec) {
        for (int i = tid * N; i < d; i += blockDim.x * N) {
            const float f = red[(i / per) * 33 + 32];
            float a[N];
            if (out1 != nullptr) {
#pragma unroll
                for (int j = 0; j < N; ++j) a[j] = row[i + j] * f * w1[i + j];
                Vec16<O>::store(out1 + i, a);
            }
            if (out2 != nullptr) {
#pragma unroll
                for (int j = 0; j < N; ++j) a[j] = row[i + j] * f * w2[i + j];
                Vec16<O>::store(out2 + i, a);
            }
        }
        return;
    }
    for (int i = tid; i < d; i += blockDim.x) {
        const float v = row[i] * red[(i / per) * 33 + 32];
        if (back != nullptr) back[i] = v * w1[i];
        else if (out1 != nullptr) out1[i] = from_f32<O>(v * w1[i]);
        if (out2 != nullptr) out2[i] = from_f32<O>(v * w2[i]);
    }
}

// ------------------------------------------------------------------------------------------------------------
// out[r] = table[token] * scale + pairs[(previous * mul_prev + token * mul_cur) mod buckets]; the first token of a
// sequence takes row `buckets` of `pairs`.  The previous token of a row is the token of the row before it when that
// belongs to the same request, else the request's state `prev` (slots, int32), which the CTA of a request's first row in
// the step reads and then sets to the request's last token of the step.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
embed_pairs_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* __restrict__ tokens,
                   const int* __restrict__ positions, const int* __restrict__ row_slot, const int* __restrict__ row_last,
                   int* __restrict__ prev, float* __restrict__ out, int d, float scale, int buckets, long long mul_prev,
                   long long mul_cur) {
    __shared__ int pair_row;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int slot = row_slot[r], tok = tokens[r];
    const T* src = table + (size_t)tok * d;
    float* dst = out + (size_t)r * d;
    if (slot < 0) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
        return;
    }
    if (threadIdx.x == 0) {
        const bool first_of_request = !(r > 0 && row_slot[r - 1] == slot);
        int before = -1;
        if (!first_of_request) before = tokens[r - 1];
        else if (positions[r] > 0) before = prev[slot];
        if (first_of_request) prev[slot] = tokens[row_last[r]];
        pair_row = before < 0 ? buckets : (int)(((long long)before * mul_prev + (long long)tok * mul_cur) % (long long)buckets);
    }
    __syncthreads();
    const T* add = pairs + (size_t)pair_row * d;
    constexpr int N = Vec16<T>::N;
    if (d % N == 0) {
        for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
            float v[N], a[N];
            Vec16<T>::load(src + i, v);
            Vec16<T>::load(add + i, a);
#pragma unroll
            for (int j = 0; j < N; ++j) dst[i + j] = fmaf(v[j], scale, a[j]);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = fmaf(to_f32(src[i]), scale, to_f32(add[i]));
    }
}

// ------------------------------------------------------------------------------------------------------------
// residual += delta_a + delta_b (each null: none); then, part by part, normed = residual * rsqrt(mean(part^2) + eps);
// out1 = normed * w1, out2 = normed * w2 (out2 null: none); in_place: residual = normed * w1 instead of out1.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_kernel(float* __restrict__ res, const T* __restrict__ delta_a, const T* __restrict__ delta_b, int groups, float eps,
                  const float* __restrict__ w1, T* __restrict__ out1, const float* __restrict__ w2, T* __restrict__ out2,
                  int in_place, int d) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[FEW_GROUPS * 33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * d;
    constexpr int N = Vec16<T>::N;
    const bool any = delta_a != nullptr || delta_b != nullptr;
    if (d % N == 0 && (((uintptr_t)res | (uintptr_t)delta_a | (uintptr_t)delta_b) % 16) == 0) {
        for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
            float v[N], dv[N];
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 x = *reinterpret_cast<const float4*>(res + base + i + j);
                v[j] = x.x; v[j + 1] = x.y; v[j + 2] = x.z; v[j + 3] = x.w;
            }
            if (delta_a != nullptr) {
                Vec16<T>::load(delta_a + base + i, dv);
#pragma unroll
                for (int j = 0; j < N; ++j) v[j] += dv[j];
            }
            if (delta_b != nullptr) {
                Vec16<T>::load(delta_b + base + i, dv);
#pragma unroll
                for (int j = 0; j < N; ++j) v[j] += dv[j];
            }
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                if (any && !in_place)
                    *reinterpret_cast<float4*>(res + base + i + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                *reinterpret_cast<float4*>(row + i + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = res[base + i];
            if (delta_a != nullptr) v += to_f32(delta_a[base + i]);
            if (delta_b != nullptr) v += to_f32(delta_b[base + i]);
            if (any && !in_place) res[base + i] = v;
            row[i] = v;
        }
    }
    __syncthreads();
    if (w1 == nullptr) return;
    grouped_norm_write<T>(row, d, groups, eps, w1, out1 != nullptr ? out1 + base : nullptr, w2,
                          out2 != nullptr ? out2 + base : nullptr, in_place ? res + base : nullptr, red);
}

// ------------------------------------------------------------------------------------------------------------
// A row of `qk` holds H query heads and then G key heads of `dim` elements.  The first `rot` elements of every head are
// rotated by the row's position, element i paired with element i + rot / 2 (cos, sin: [positions][rot / 2]); queries in
// place, keys on their way into the key rows of the row's page; the keys as they were projected go into the value rows.
// Pages: element (page, kv head, position in the page, i) at pages + page * page_stride + head * head_stride +
// position * dim + i.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rotate_tie_store_kernel(T* __restrict__ qk, int ld, int H, int G, int dim, int rot, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, T* __restrict__ k_pages, size_t k_page_stride, size_t k_head_stride,
                        T* __restrict__ v_pages, size_t v_page_stride, size_t v_head_stride, int page_size, int num_pages,
                        const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                        const int* __restrict__ row_slot, int* __restrict__ fault) {
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    const int half = rot >> 1;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    pdl_wait();
    T* row = qk + (size_t)r * ld;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        T* q = row + (size_t)h * dim;
        const float a = to_f32(q[i]), b = to_f32(q[i + half]);
        q[i] = from_f32<T>(a * cs[i] - b * sn[i]);
        q[i + half] = from_f32<T>(b * cs[i] + a * sn[i]);
    }
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(fault, 5);
        return;
    }
    const int in_page = pos % page_size;
    const T* keys = row + (size_t)H * dim;
    for (int idx = threadIdx.x; idx < G * dim; idx += blockDim.x) {
        const int g = idx / dim, e = idx - g * dim;
        const T* k = keys + (size_t)g * dim;
        const T raw = k[e];
        T turned = raw;
        if (e < rot) {
            const int i = e < half ? e : e - half;
            const float a = to_f32(k[i]), b = to_f32(k[i + half]);
            turned = from_f32<T>(e < half ? a * cs[i] - b * sn[i] : b * cs[i] + a * sn[i]);
        }
        k_pages[(size_t)page * k_page_stride + (size_t)g * k_head_stride + (size_t)in_page * dim + e] = turned;
        v_pages[(size_t)page * v_page_stride + (size_t)g * v_head_stride + (size_t)in_page * dim + e] = raw;
    }
}

// ------------------------------------------------------------------------------------------------------------
// y = (o_raw + skip[head] * x) * silu(z) over a row of H heads of v_dim elements; then the row in `groups` equal parts,
// each divided by its root mean square (eps inside the root), times w.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
skip_gate_group_norm_kernel(const float* __restrict__ o_raw, const T* __restrict__ x, int ldx, const float* __restrict__ skip,
                            const T* __restrict__ z, int ldz, const float* __restrict__ w, int groups, float eps,
                            T* __restrict__ out, int ldo, const int* __restrict__ row_slot, int H, int v_dim) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[FEW_GROUPS * 33];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    if (row_slot[r] < 0) return;
    pdl_wait();
    const int d = H * v_dim;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float zz = to_f32(z[(size_t)r * ldz + i]);
        const float y = fmaf(skip[i / v_dim], to_f32(x[(size_t)r * ldx + i]), o_raw[(size_t)r * d + i]);
        row[i] = y * (zz / (1.f + expf(-zz)));
    }
    __syncthreads();
    grouped_norm_write<T>(row, d, groups, eps, w, out + (size_t)r * ldo, nullptr, (T*)nullptr, nullptr, red);
}

// out = a * sa + b * sb, element by element over n rows of d (row strides free), the sum in 32-bit.
template <typename T>
__global__ void __launch_bounds__(256)
scaled_sum_kernel(const T* __restrict__ a, int lda, float sa, const T* __restrict__ b, int ldb, float sb, T* __restrict__ out,
                  int ldo, int d, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / d;
        const int j = (int)(idx - r * d);
        out[r * ldo + j] = from_f32<T>(fmaf(to_f32(a[r * lda + j]), sa, to_f32(b[r * ldb + j]) * sb));
    }
}

}  // namespace

TIS_API int tis_embed_pairs(int dtype, const void* table, const void* pairs, const int* tokens, const int* positions,
                            const int* row_slot, const int* row_last, int* prev, float* out, int n, int d, float scale,
                            int buckets, long long mul_prev, long long mul_cur, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (buckets <= 0 || d <= 0) {
        tis_set_error("embed_pairs: %d buckets, width %d", buckets, d);
        return TIS_BAD_SIZE;
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(embed_pairs_kernel<T>, dim3(n), dim3(256), 0, stream, (const T*)table, (const T*)pairs, tokens, positions,
                   row_slot, row_last, prev, out, d, scale, buckets, mul_prev, mul_cur));
    return tis_check_launch("embed_pairs");
}

TIS_API int tis_group_norm(int dtype, float* residual, const void* delta_a, const void* delta_b, int groups, float eps,
                           const float* w1, void* out1, const float* w2, void* out2, int in_place, int n, int d,
                           cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (groups <= 0 || d <= 0 || d % groups || (size_t)d * sizeof(float) > 96 * 1024 || (out2 != nullptr && w2 == nullptr) ||
        (w1 == nullptr && (out1 != nullptr || in_place))) {
        tis_set_error("group_norm: width %d in %d groups (one row must fit 96 KB of shared memory)", d, groups);
        return TIS_BAD_SIZE;
    }
    const size_t smem = (size_t)d * sizeof(float);
    TIS_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(group_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tis_launch(group_norm_kernel<T>, dim3(n), dim3(256), smem, stream, residual, (const T*)delta_a, (const T*)delta_b, groups,
                   eps, w1, (T*)out1, w2, (T*)out2, in_place, d);
    });
    return tis_check_launch("group_norm");
}

TIS_API int tis_rotate_tie_store(int dtype, void* qk, int ld, int H, int G, int dim, int rot, const float* cos_t,
                                 const float* sin_t, void* k_pages, size_t k_page_stride, size_t k_head_stride, void* v_pages,
                                 size_t v_page_stride, size_t v_head_stride, int page_size, int num_pages,
                                 const int* block_table, int bt_stride, const int* positions, const int* row_slot, int* fault,
                                 int n, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (H <= 0 || G <= 0 || dim <= 0 || rot < 0 || rot % 2 || rot > dim || page_size <= 0) {
        tis_set_error("rotate_tie_store: %d heads, %d kv heads of %d elements, %d of them rotated", H, G, dim, rot);
        return TIS_BAD_SIZE;
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(rotate_tie_store_kernel<T>, dim3(n), dim3(128), 0, stream, (T*)qk, ld, H, G, dim, rot, cos_t, sin_t,
                   (T*)k_pages, k_page_stride, k_head_stride, (T*)v_pages, v_page_stride, v_head_stride, page_size, num_pages,
                   block_table, bt_stride, positions, row_slot, fault));
    return tis_check_launch("rotate_tie_store");
}

TIS_API int tis_skip_gate_group_norm(int dtype, const float* o_raw, const void* x, int ldx, const float* skip, const void* z,
                                     int ldz, const float* w, int groups, float eps, void* out, int ldo, const int* row_slot,
                                     int n, int H, int v_dim, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    const int d = H * v_dim;
    if (groups <= 0 || d <= 0 || d % groups || (size_t)d * sizeof(float) > 96 * 1024) {
        tis_set_error("skip_gate_group_norm: %d heads of %d in %d groups", H, v_dim, groups);
        return TIS_BAD_SIZE;
    }
    const size_t smem = (size_t)d * sizeof(float);
    TIS_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(skip_gate_group_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tis_launch(skip_gate_group_norm_kernel<T>, dim3(n), dim3(256), smem, stream, o_raw, (const T*)x, ldx, skip, (const T*)z,
                   ldz, w, groups, eps, (T*)out, ldo, row_slot, H, v_dim);
    });
    return tis_check_launch("skip_gate_group_norm");
}

TIS_API int tis_scaled_sum(int dtype, const void* a, int lda, float sa, const void* b, int ldb, float sb, void* out, int ldo,
                           int n, int d, cudaStream_t stream) {
    if (n <= 0 || d <= 0) return TIS_OK;
    const size_t total = (size_t)n * d;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(scaled_sum_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)a, lda, sa, (const T*)b, ldb, sb, (T*)out,
                   ldo, d, total));
    return tis_check_launch("scaled_sum");
}
