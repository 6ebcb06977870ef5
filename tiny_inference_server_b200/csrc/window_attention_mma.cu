// Attention over a window of the paged cache on the tensor cores (bfloat16, mma.sync m16n8k16), for keys of
// TIS_KD and values of TIS_VD elements (compiled per pair of widths):
//   score = q . k * scale - r1[head] * ln(1 + r2[head] * distance),  keys pos - window < j <= pos,
//   softmax in 32-bit, out = softmax . v * sigmoid(gate).
// A CTA takes one tile of consecutive rows of one request and one kv head, with all the query heads that share
// the kv head: row r and query head h of the group are packed row r * (H / G) + h of a block of 64 packed rows, so
// that a key or value row is brought into shared memory once for all of them.  Tiles of many rows: each of the four
// warps owns 16 packed rows and walks all keys the tile can see, 64 at a time, with the running maximum and sum of
// its rows in registers.  Tiles of at most 16 packed rows (decode rows): the four warps share the rows and take
// every fourth tile of keys each; their partial results are merged through shared memory.  Key and value rows are
// copied from their pages by cp.async, two tiles in flight.  The key tiles of decode rows may also be shared out over
// several CTAs (grid.z), whose partial results a second small kernel merges.  Scores, bias, maximum, sum and the output are 32-bit;
// the probabilities enter the second product rounded to bfloat16.
#include "common.cuh"

#ifndef TIS_KD
#define TIS_KD 64
#endif
#ifndef TIS_VD
#define TIS_VD 64
#endif

namespace {

constexpr int KD = TIS_KD, VD = TIS_VD;
static_assert(KD % 16 == 0 && VD % 16 == 0, "key width and value width must be multiples of 16");
constexpr int ROWS = 64, KEYS = 64, THREADS = 128;       // ROWS == KEYS: the queries fit a key stage
constexpr int MIN_CTAS = KD + VD <= 256 ? 3 : 1;          // CTAs an SM that the register budget is set for
constexpr int QS = KD + 8, KS = KD + 8, VS = VD + 8;       // row strides in shared memory (elements): no bank conflicts

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

struct Params {
    const bf16* q; int ldq;
    const bf16* gate; int ldg;
    int gate_per_head;       // `gate` holds one number per query head (for all its elements) instead of one per element
    bf16* out; int ldo;
    const bf16* k_pages; size_t k_page_stride, k_head_stride;
    const bf16* v_pages; size_t v_page_stride, v_head_stride;
    const int* block_table; int bt_stride; int num_pages;
    const int* positions; const int* row_slot;
    const int* tile_row0; const int* tile_rows;
    int H, G, page_size, window;
    float scale;
    const float* r1; const float* r2;
    const float* sink;       // per query head: exp(sink) is one more term of the softmax's denominator (null: none)
    int v_row;               // elements from one value row of a page to the next (VD, or more when the rows are slices)
    int* fault;
    float* partial;          // [tiles][G][splits][64][VD + 2]: unnormalised out, maximum, sum (key splits over CTAs)
};

// Copies the key and value rows first .. first + 63 (those that exist: j <= last) of a request into a stage.  Two
// threads share a key: one look-up of its page, then every other 16-byte chunk of its two rows each.
__device__ __forceinline__ void load_tile(const Params& p, int slot, int kvh, int first, int last, bf16* ks, bf16* vs,
                                          int* bad) {
    constexpr int KC = KD / 8, VC = VD / 8;
    static_assert(THREADS == 2 * KEYS, "two threads a key");
    const int key = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int j = first + key;
    bf16* kd = ks + key * KS;
    bf16* vd = vs + key * VS;
    int page = -1;
    if (j <= last) {
        page = p.block_table[(size_t)slot * p.bt_stride + j / p.page_size];
        if (page < 0 || page >= p.num_pages) { *bad = 1; page = -1; }
    }
    if (page >= 0) {
        const int in_page = j % p.page_size;
        const bf16* ksrc = p.k_pages + (size_t)page * p.k_page_stride + (size_t)kvh * p.k_head_stride + (size_t)in_page * KD;
        const bf16* vsrc = p.v_pages + (size_t)page * p.v_page_stride + (size_t)kvh * p.v_head_stride + (size_t)in_page * p.v_row;
#pragma unroll
        for (int c = 0; c < KC / 2; ++c) cp_async16(kd + (2 * c + half) * 8, ksrc + (2 * c + half) * 8);
#pragma unroll
        for (int c = 0; c < VC / 2; ++c) cp_async16(vd + (2 * c + half) * 8, vsrc + (2 * c + half) * 8);
    } else {                                                  // keys that do not exist: finite zeros
#pragma unroll
        for (int c = 0; c < KC / 2; ++c) *reinterpret_cast<uint4*>(kd + (2 * c + half) * 8) = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int c = 0; c < VC / 2; ++c) *reinterpret_cast<uint4*>(vd + (2 * c + half) * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
}

__global__ void __launch_bounds__(THREADS, MIN_CTAS)
window_attention_mma_kernel(const Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int bad;
    bf16* kbuf = reinterpret_cast<bf16*>(smem_raw);            // [2][KEYS][KS]
    bf16* vbuf = kbuf + 2 * KEYS * KS;                         // [2][KEYS][VS]
    bf16* qs = kbuf + KEYS * KS;                               // [ROWS][QS]: the queries pass through the second key stage
    pdl_launch_dependents();
    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int row0 = p.tile_row0[tile], nrows = p.tile_rows[tile];
    const int slot = p.row_slot[row0];
    if (slot < 0 || nrows <= 0) return;
    const int pos0 = p.positions[row0];
    const int gq = p.H / p.G;                                  // query heads that share the kv head
    const int packed = nrows * gq;                             // packed rows in use (<= 64)
    const bool split_keys = packed <= 16;                      // the warps share the rows and split the key tiles
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    if (tid == 0) bad = 0;
    const int last = pos0 + nrows - 1;                         // the last key any row of the tile sees
    const int first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    int ntiles = (last - first) / KEYS + 1;
    int kt_begin = 0;
    const int splits = gridDim.z;
    if (splits > 1) {
        // the key tiles of a tile of rows are shared out over the CTAs of grid.z (a decode step: few tiles, each with
        // many keys to walk), whose partial results the merge kernel adds up
        const int per = (ntiles + splits - 1) / splits;
        kt_begin = min(ntiles, (int)blockIdx.z * per);
        ntiles = min(ntiles, kt_begin + per);
    }
    const int base = split_keys ? 0 : warp * 16;               // first packed row of this warp
    // this thread's two packed rows: base + g and base + g + 8
    const int m_a = base + g, m_b = m_a + 8;
    const bool row_a = m_a < packed, row_b = m_b < packed;
    const int pos_a = pos0 + m_a / gq, pos_b = pos0 + m_b / gq;
    const int head_a = kvh * gq + m_a % gq, head_b = kvh * gq + m_b % gq;
    float b1_a = 0.f, b2_a = 0.f, b1_b = 0.f, b2_b = 0.f;
    if (p.r1 != nullptr) {
        if (row_a) { b1_a = p.r1[head_a]; b2_a = p.r2[head_a]; }
        if (row_b) { b1_b = p.r1[head_b]; b2_b = p.r2[head_b]; }
    }
    pdl_wait();
    // queries of the tile (packed rows beyond those in use: zeros)
    for (int idx = tid; idx < ROWS * (KD / 8); idx += THREADS) {
        const int m = idx / (KD / 8), c = idx - m * (KD / 8);
        bf16* dst = qs + m * QS + c * 8;
        if (m < packed) cp_async16(dst, p.q + (size_t)(row0 + m / gq) * p.ldq + (size_t)(kvh * gq + m % gq) * KD + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();                                           // `bad` is initialised before any load may set it
    if (kt_begin < ntiles) load_tile(p, slot, kvh, first + kt_begin * KEYS, last, kbuf, vbuf, &bad);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    unsigned qf[KD / 16][4];
#pragma unroll
    for (int kk = 0; kk < KD / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (base + (lane & 7) + 8 * ((lane >> 3) & 1)) * QS + kk * 16 + 8 * (lane >> 4));
    __syncthreads();                                           // the queries are in registers: the stage is free
    float o[VD / 8][4];
#pragma unroll
    for (int n = 0; n < VD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    if (p.sink != nullptr && !split_keys && blockIdx.z == 0) {
        // the sink's term: the running maximum starts at the sink and the running sum at 1 (in one of the four
        // threads that share a row); it counts once, with the first share of the keys.  Rows whose keys the four warps
        // share get it when those merge.
        if (row_a) { m[0] = p.sink[head_a]; l[0] = t4 == 0 ? 1.f : 0.f; }
        if (row_b) { m[1] = p.sink[head_b]; l[1] = t4 == 0 ? 1.f : 0.f; }
    }
    // positions of the first and last row among this warp's packed rows
    const int w_lo = pos0 + base / gq, w_hi = min(pos0 + (base + 15) / gq, last);
    for (int kt = kt_begin; kt < ntiles; ++kt) {
        const int stage = (kt - kt_begin) & 1;
        if (kt + 1 < ntiles)
            load_tile(p, slot, kvh, first + (kt + 1) * KEYS, last, kbuf + (stage ^ 1) * KEYS * KS, vbuf + (stage ^ 1) * KEYS * VS, &bad);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* ks = kbuf + stage * KEYS * KS;
        const bf16* vs = vbuf + stage * KEYS * VS;
        const int j0 = first + kt * KEYS;
        // does this warp see any key of the tile?
        bool any = base < packed && j0 <= w_hi && (p.window <= 0 || j0 + KEYS - 1 > w_lo - p.window);
        if (split_keys) any = any && (kt & 3) == warp;
        if (any) {
            float s[KEYS / 8][4];
#pragma unroll
            for (int n = 0; n < KEYS / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < KD / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < KEYS / 16; ++n2) {
                    unsigned b[4];
                    ldmatrix_x4(b, ks + (n2 * 16 + (lane & 7) + 8 * (lane >> 4)) * KS + kk * 16 + 8 * ((lane >> 3) & 1));
                    mma_bf16(s[2 * n2], qf[kk], b[0], b[1]);
                    mma_bf16(s[2 * n2 + 1], qf[kk], b[2], b[3]);
                }
            }
            // scale, bias, mask; the maximum of each row over the tile.  A tile that every row of the warp sees
            // whole (the usual case inside a window) needs no mask.
            const bool whole = base + 15 < packed && j0 + KEYS - 1 <= w_lo && (p.window <= 0 || j0 > w_hi - p.window);
            float mx[2] = {-INFINITY, -INFINITY};
            if (whole) {
#pragma unroll
                for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + n * 8 + 2 * t4 + (e & 1);
                        const int pos = (e & 2) ? pos_b : pos_a;
                        const float v = s[n][e] * p.scale - ((e & 2) ? b1_b : b1_a) * __logf(fmaf((e & 2) ? b2_b : b2_a, (float)(pos - j), 1.f));
                        s[n][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
            } else {
#pragma unroll
                for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + n * 8 + 2 * t4 + (e & 1);
                        const int pos = (e & 2) ? pos_b : pos_a;
                        const bool ok = ((e & 2) ? row_b : row_a) && j <= pos && (p.window <= 0 || j > pos - p.window);
                        float v = -INFINITY;
                        if (ok) v = s[n][e] * p.scale - ((e & 2) ? b1_b : b1_a) * __logf(fmaf((e & 2) ? b2_b : b2_a, (float)(pos - j), 1.f));
                        s[n][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
            }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m[h], mx[h]);
                corr[h] = m[h] == -INFINITY ? 0.f : __expf(m[h] - m_new);
                m[h] = m_new;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float mm = m[e >> 1];
                    const float pv = (s[n][e] == -INFINITY || mm == -INFINITY) ? 0.f : __expf(s[n][e] - mm);
                    s[n][e] = pv;
                    sum[e >> 1] += pv;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) l[h] = l[h] * corr[h] + sum[h];
#pragma unroll
            for (int n = 0; n < VD / 8; ++n) {
                o[n][0] *= corr[0]; o[n][1] *= corr[0];
                o[n][2] *= corr[1]; o[n][3] *= corr[1];
            }
            // out += P . V
#pragma unroll
            for (int kk = 0; kk < KEYS / 16; ++kk) {
                unsigned pa[4];
#pragma unroll
                for (int a = 0; a < 4; ++a)
                    pa[a] = pack_bf16(s[2 * kk + (a >> 1)][(a & 1) * 2], s[2 * kk + (a >> 1)][(a & 1) * 2 + 1]);
#pragma unroll
                for (int n2 = 0; n2 < VD / 16; ++n2) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * VS + n2 * 16 + 8 * (lane >> 4));
                    mma_bf16(o[2 * n2], pa, b[0], b[1]);
                    mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                       // the stage may be loaded again
    }
    cp_async_wait<0>();
    if (bad && tid == 0) atomicExch(p.fault, 5);
    // the sums of a row lie in the four threads that share it
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    if (split_keys) {
        // merge the four warps' partial results of the 16 packed rows (the key and value stages are free now)
        float* part = reinterpret_cast<float*>(kbuf);          // [4 warps][16 rows][VD + 2]: out, maximum, sum
        constexpr int PS = VD + 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* dst = part + ((size_t)warp * 16 + g + 8 * h) * PS;
#pragma unroll
            for (int n = 0; n < VD / 8; ++n) {
                dst[n * 8 + 2 * t4] = o[n][2 * h];
                dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
            }
            if (t4 == 0) { dst[VD] = m[h]; dst[VD + 1] = l[h]; }
        }
        __syncthreads();
        for (int idx = tid; idx < packed * VD; idx += THREADS) {
            const int mrow = idx / VD, c = idx - mrow * VD;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, part[((size_t)w * 16 + mrow) * PS + VD]);
            float num = 0.f, den = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* src = part + ((size_t)w * 16 + mrow) * PS;
                const float f = src[VD] == -INFINITY ? 0.f : __expf(src[VD] - mm);
                num = fmaf(src[c], f, num);
                den = fmaf(src[VD + 1], f, den);
            }
            if (p.sink != nullptr && blockIdx.z == 0) {        // the sink's term counts once: with the first share of the keys
                const float sk = p.sink[kvh * gq + mrow % gq];
                const float m2 = fmaxf(mm, sk);
                const float f = mm == -INFINITY ? 0.f : __expf(mm - m2);
                num *= f;
                den = fmaf(den, f, __expf(sk - m2));
                mm = m2;
            }
            if (splits > 1) {                                  // this CTA's share of the keys: left for the merge kernel
                float* dst = p.partial + ((((size_t)tile * p.G + kvh) * splits + blockIdx.z) * ROWS + mrow) * PS;
                dst[c] = num;
                if (c == 0) { dst[VD] = mm; dst[VD + 1] = den; }
                continue;
            }
            float x = den > 0.f ? num / den : 0.f;
            const size_t row = (size_t)(row0 + mrow / gq);
            const size_t col = (size_t)(kvh * gq + mrow % gq) * VD + c;
            if (p.gate != nullptr)
                x = x / (1.f + __expf(-__bfloat162float(p.gate[row * p.ldg + (p.gate_per_head ? (size_t)(kvh * gq + mrow % gq) : col)])));
            p.out[row * p.ldo + col] = __float2bfloat16_rn(x);
        }
        return;
    }
    if (splits > 1) {                                          // this CTA's share of the keys: left for the merge kernel
        constexpr int PS = VD + 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int mrow = base + g + 8 * h;
            if (mrow >= packed) continue;
            float* dst = p.partial + ((((size_t)tile * p.G + kvh) * splits + blockIdx.z) * ROWS + mrow) * PS;
#pragma unroll
            for (int n = 0; n < VD / 8; ++n) {
                dst[n * 8 + 2 * t4] = o[n][2 * h];
                dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
            }
            if (t4 == 0) { dst[VD] = m[h]; dst[VD + 1] = l[h]; }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int mrow = base + g + 8 * h;
        if (mrow >= packed) continue;
        const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        const size_t row = (size_t)(row0 + mrow / gq);
        const size_t col0 = (size_t)(kvh * gq + mrow % gq) * VD;
#pragma unroll
        for (int n = 0; n < VD / 8; ++n) {
            const int c = n * 8 + 2 * t4;
            float x0 = o[n][2 * h] * inv, x1 = o[n][2 * h + 1] * inv;
            if (p.gate != nullptr && p.gate_per_head) {
                const float gh = 1.f / (1.f + __expf(-__bfloat162float(p.gate[row * p.ldg + kvh * gq + mrow % gq])));
                x0 *= gh;
                x1 *= gh;
            } else if (p.gate != nullptr) {
                const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(p.gate + row * p.ldg + col0 + c);
                x0 = x0 / (1.f + __expf(-__bfloat162float(gv.x)));
                x1 = x1 / (1.f + __expf(-__bfloat162float(gv.y)));
            }
            *reinterpret_cast<__nv_bfloat162*>(p.out + row * p.ldo + col0 + c) = __floats2bfloat162_rn(x0, x1);
        }
    }
}

// The key splits of a tile, merged: a CTA per (tile, kv head, packed row).  The splits' maxima and sums of the row
// are read once, by a thread each, and turned into one factor per split in shared memory; then a thread per output
// column adds up the splits' partial outputs with those factors.
__global__ void __launch_bounds__(128)
window_attention_merge_kernel(const Params p, int splits) {
    __shared__ float factor[64];
    __shared__ float red[33];
    pdl_launch_dependents();
    const int tile = blockIdx.x, kvh = blockIdx.y, mrow = blockIdx.z;
    const int row0 = p.tile_row0[tile], nrows = p.tile_rows[tile];
    const int gq = p.H / p.G;
    const int packed = nrows * gq;
    if (nrows <= 0 || p.row_slot[row0] < 0 || mrow >= packed) return;
    pdl_wait();
    constexpr int PS = VD + 2;
    const float* part = p.partial + ((((size_t)tile * p.G + kvh) * splits) * ROWS + mrow) * PS;
    const size_t step = (size_t)ROWS * PS;               // from one split's row to the next split's
    const int tid = threadIdx.x;
    float m_s = -INFINITY, l_s = 0.f;
    if (tid < splits) { m_s = part[tid * step + VD]; l_s = part[tid * step + VD + 1]; }
    const float mm = block_max(m_s, red);
    const float f = (tid < splits && m_s != -INFINITY) ? __expf(m_s - mm) : 0.f;
    if (tid < 64) factor[tid] = f;
    const float den = block_sum(l_s * f, red);            // its barriers also publish the factors
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const size_t row = (size_t)(row0 + mrow / gq);
    for (int c = tid; c < VD; c += blockDim.x) {
        float num = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) num = fmaf(part[s * step + c], factor[s], num);
        float x = num * inv;
        const size_t col = (size_t)(kvh * gq + mrow % gq) * VD + c;
        if (p.gate != nullptr)
            x = x / (1.f + __expf(-__bfloat162float(p.gate[row * p.ldg + (p.gate_per_head ? (size_t)(kvh * gq + mrow % gq) : col)])));
        p.out[row * p.ldo + col] = __float2bfloat16_rn(x);
    }
}

}  // namespace

// Floats of scratch that `splits` key splits of `num_tiles` tiles need.
TIS_API size_t tis_window_attention_partial_floats(int num_tiles, int G, int splits) {
    return (size_t)num_tiles * G * splits * ROWS * (VD + 2);
}

TIS_API int tis_window_attention_mma_dims(int* kd, int* vd) {
    *kd = KD;
    *vd = VD;
    return TIS_OK;
}

// Tiles hold at most 64 / (H / G) rows.  Rows of q, gate and out must start on 16-byte (q) and 4-byte (gate, out) boundaries: ldq a multiple of 8,
// ldg and ldo even; page rows on 16-byte boundaries (strides multiples of 8 elements).
TIS_API int tis_window_attention_mma(const void* q, int ldq, const void* gate, int ldg, void* out, int ldo,
                                     const void* k_pages, size_t k_page_stride, size_t k_head_stride,
                                     const void* v_pages, size_t v_page_stride, size_t v_head_stride,
                                     const int* block_table, int bt_stride, int num_pages, const int* positions,
                                     const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                                     int H, int G, int page_size, int window, float scale, const float* r1,
                                     const float* r2, int splits, float* partial, const float* sink, int v_row,
                                     int gate_per_head, int* fault, cudaStream_t stream) {
    if (num_tiles <= 0) return TIS_OK;
    if (splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) {
        tis_set_error("window_attention_mma: %d key splits%s", splits, splits > 1 ? " without scratch" : "");
        return TIS_BAD_SIZE;
    }
    if (H <= 0 || G <= 0 || H % G || H / G > ROWS || page_size <= 0 || window < 0 || ldq % 8 || (ldg % 2 && !gate_per_head) ||
        ldo % 2 ||
        v_row < VD || v_row % 8 ||
        k_page_stride % 8 || k_head_stride % 8 || v_page_stride % 8 || v_head_stride % 8 ||
        ((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16 || ((gate_per_head ? (uintptr_t)0 : (uintptr_t)gate) | (uintptr_t)out) % 4) {
        tis_set_error("window_attention_mma: %d query heads, %d kv heads, page size %d, window %d, row strides %d/%d/%d "
                      "or an operand that is not aligned", H, G, page_size, window, ldq, ldg, ldo);
        return TIS_BAD_SIZE;
    }
    Params p;
    p.q = (const bf16*)q; p.ldq = ldq;
    p.gate = (const bf16*)gate; p.ldg = ldg; p.gate_per_head = gate_per_head;
    p.out = (bf16*)out; p.ldo = ldo;
    p.k_pages = (const bf16*)k_pages; p.k_page_stride = k_page_stride; p.k_head_stride = k_head_stride;
    p.v_pages = (const bf16*)v_pages; p.v_page_stride = v_page_stride; p.v_head_stride = v_head_stride;
    p.block_table = block_table; p.bt_stride = bt_stride; p.num_pages = num_pages;
    p.positions = positions; p.row_slot = row_slot; p.tile_row0 = tile_row0; p.tile_rows = tile_rows;
    p.H = H; p.G = G; p.page_size = page_size; p.window = window; p.scale = scale; p.r1 = r1; p.r2 = r2; p.fault = fault; p.partial = partial; p.sink = sink; p.v_row = v_row;
    const size_t smem = sizeof(bf16) * ((size_t)2 * KEYS * KS + 2 * KEYS * VS);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaFuncSetAttribute(window_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    tis_launch(window_attention_mma_kernel, dim3(num_tiles, G, splits), dim3(THREADS), smem, stream, p);
    int st = tis_check_launch("window_attention_mma");
    if (st != TIS_OK || splits == 1) return st;
    // a step whose keys are split holds one row a tile: H / G packed rows
    const int rows_bound = H / G < ROWS ? H / G : ROWS;
    tis_launch(window_attention_merge_kernel, dim3(num_tiles, G, rows_bound), dim3(128), 0, stream, p, splits);
    return tis_check_launch("window_attention_merge");
}
