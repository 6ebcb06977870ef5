// Between the projections and the cache of attention whose keys and values are expanded from one compressed vector
// per token (a page row holds that vector followed by one rotated key slice, shared by all heads).
// Everything is computed in 32-bit; T is the storage type of activations and pages.
#include "common.cuh"

// A row of `proj` holds, per head, flat + rot query elements, and from column dkv_at on rank + rot elements of the
// compressed projection.  Per row (a CTA):
//   * the last rot elements of every head's query are rotated by the row's position (the first `dims` of them, in pairs
//     (i, i + dims / 2) with angles from the tables cos / sin [positions][dims / 2]; the rest pass unchanged) and written to
//     q_out[row][head * (rank + rot) + rank ...];
//   * c = x[0 .. rank) * rsqrt(mean(x^2) + eps) * cw and the rotated last rot elements of the compressed projection are
//     written as the row [c | slice] of the position's page: k_pages + page * page_stride + in_page * (rank + rot).
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int dkv_at, int H, int flat, int rot, int dims, int rank,
                      const float* __restrict__ cw, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int table_rows, T* __restrict__ q_out, int ldq,
                      T* __restrict__ k_pages, size_t page_stride, int page_size, int num_pages,
                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                      const int* __restrict__ row_slot, int* __restrict__ fault) {
    __shared__ float red[33];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = positions[r];
    const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
    const int half = dims / 2, rest = rot - dims, tid = threadIdx.x, nthr = blockDim.x;
    if (pos < 0 || (dims > 0 && pos >= table_rows) || page < 0 || page >= num_pages) {
        if (tid == 0) atomicExch(fault, 6);
        return;
    }
    const float* cs = dims > 0 ? cos_t + (size_t)pos * half : nullptr;     // rot 0: nothing is rotated, the tables may be null
    const float* sn = dims > 0 ? sin_t + (size_t)pos * half : nullptr;
    pdl_wait();
    const T* row = proj + (size_t)r * ld;
    const int qd = flat + rot, rw = rank + rot;
    for (int idx = tid; idx < H * half; idx += nthr) {
        const int h = idx / half, i = idx - h * half;
        const float a = to_f32(row[h * qd + flat + i]), b = to_f32(row[h * qd + flat + half + i]);
        const float c = cs[i], s = sn[i];
        T* dst = q_out + (size_t)r * ldq + (size_t)h * rw + rank;
        dst[i] = from_f32<T>(a * c - b * s);
        dst[half + i] = from_f32<T>(b * c + a * s);
    }
    for (int idx = tid; idx < H * rest; idx += nthr) {       // the channels of the slice that are not rotated
        const int h = idx / rest, i = dims + idx - h * rest;
        q_out[(size_t)r * ldq + (size_t)h * rw + rank + i] = row[h * qd + flat + i];
    }
    const T* low = row + dkv_at;
    float ss = 0.f;
    for (int i = tid; i < rank; i += nthr) { const float v = to_f32(low[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float f = rsqrtf(ss / (float)rank + eps);
    T* dst = k_pages + (size_t)page * page_stride + (size_t)(pos % page_size) * rw;
    for (int i = tid; i < rank; i += nthr) dst[i] = from_f32<T>(to_f32(low[i]) * f * cw[i]);
    for (int i = tid; i < half; i += nthr) {
        const float a = to_f32(low[rank + i]), b = to_f32(low[rank + half + i]);
        const float c = cs[i], s = sn[i];
        dst[rank + i] = from_f32<T>(a * c - b * s);
        dst[rank + half + i] = from_f32<T>(b * c + a * s);
    }
    for (int i = dims + tid; i < rot; i += nthr) dst[rank + i] = low[rank + i];
}

TIS_API int tis_latent_prepare(int dtype, const void* proj, int ld, int dkv_at, int H, int flat, int rot, int dims, int rank,
                               const float* cw, float eps, const float* cos_t, const float* sin_t, int table_rows,
                               void* q_out, int ldq, void* k_pages, size_t page_stride, int page_size, int num_pages,
                               const int* block_table, int bt_stride, const int* positions, const int* row_slot,
                               int* fault, int n, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (H <= 0 || flat < 0 || rot < 0 || dims < 0 || dims % 2 || dims > rot || rank <= 0 || page_size <= 0 ||
        dkv_at < H * (flat + rot) || (dims > 0 && (cos_t == nullptr || sin_t == nullptr))) {
        tis_set_error("latent_prepare: %d heads, %d + %d query elements a head of which %d rotated, rank %d, page size %d", H,
                      flat, rot, dims, rank, page_size);
        return TIS_BAD_SIZE;
    }
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(latent_prepare_kernel<T>, dim3(n), dim3(128), 0, stream, (const T*)proj, ld, dkv_at, H, flat, rot, dims,
                   rank, cw, eps, cos_t, sin_t, table_rows, (T*)q_out, ldq, (T*)k_pages, page_stride, page_size, num_pages,
                   block_table, bt_stride, positions, row_slot, fault));
    return tis_check_launch("latent_prepare");
}
