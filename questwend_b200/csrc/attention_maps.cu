// Attention over the paged cache with one or two score maps per head, soft-capped scores and a causal or chunked mask.
//
// A query head has `maps` (1 or 2) query vectors of `dim` values, laid out one after the other, and so has a key head;
// map m of query head h is scored against map m of key head h / (H / G).  Each map is a softmax attention of its own
// over the SAME values (size vdim).  With two maps the head's output is their difference, a1 - lambda * a2 (differential
// attention; lambda is one number for the layer); with `norm_out` the output is then divided by its root mean square
// over vdim (eps inside the root) and multiplied by out_scale.
//   score = q . k * scale;  softcap > 0:  score <- softcap * tanh(score / softcap)
//   mask:  key j is seen from position p when j <= p and (chunk > 0) floor(j / chunk) = floor(p / chunk); chunks are
//          counted from position 0 of the sequence.
// Scores, maxima, sums, accumulators, the difference and the norm are 32-bit; q and the cache are float or bfloat16.
// The cache: K pool [pages, G, 64, maps * dim], V pool [pages, G, 64, vdim].
//
//   maps_prep         bias, per-map RMS norm of q and k (a weight of dim values shared by heads and maps), rotation of the
//                     first rdims values of every map of q and k, cache write of a step's tokens; q out
//   maps_prefill      any number of new tokens per sequence (float and bfloat16, any sizes up to 256)
//   maps_prefill_mma  bfloat16 prompts on the tensor cores
//   maps_decode       one new token per sequence: runs of pages, one block of threads a run, then maps_merge, which also
//                     takes the difference and the norm
#include "common.cuh"

#define QWB_MAPS_MAX_DIM 256
#define QWB_MAPS_PAGE 64
#define QWB_MAPS_MAX 2
#define QWB_MAPS_ROWS 8           // (query head, map) pairs per block of the decode kernel (even: see its score loop)
#define QWB_MAPS_RUN_PAGES 2      // pages per run of the decode kernel, doubled while a sequence would have more than ...
#define QWB_MAPS_MAX_RUNS 64      // ... this many runs: follows from the sequence's own length, not from the batch

// value i of a vector after its first n values were turned by the angle whose cos and sin are cs[m], sn[m] for pair m
__device__ __forceinline__ float maps_turned(const float* v, int i, int n, const float* cs, const float* sn, int interleaved) {
    if (i >= n) return v[i];
    const int half = n >> 1;
    int m, first;
    float a, b;
    if (interleaved) { m = i >> 1; first = !(i & 1); a = v[2 * m]; b = v[2 * m + 1]; }
    else { m = i < half ? i : i - half; first = i < half; a = v[m]; b = v[m + half]; }
    const float c = cs[m], s = sn[m];
    return first ? a * c - b * s : b * c + a * s;
}

__device__ __forceinline__ int maps_first_key(int p, int chunk) { return chunk > 0 ? (p / chunk) * chunk : 0; }

__device__ __forceinline__ float maps_cap(float s, float cap, float inv_cap) { return cap > 0.f ? cap * tanhf(s * inv_cap) : s; }

// ---------------------------------------------------------------------------------
// prep: grid (T, ceil(items / 4)), 4 warps, a warp per (token, item); items = H * maps query maps, G * maps key maps,
// G values.  qkv [T, (H + G) * maps * dim + G * vdim] float: the projections (after a convolution, if the mixer has one).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void maps_prep_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, const float* __restrict__ qw,
                                 const float* __restrict__ kw, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                 int table_width, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, int H, int G,
                                 int maps, int dim, int vdim, int rdims, int interleaved, float eps, int store_kv) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float bufs[4][QWB_MAPS_MAX_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y * 4 + warp, t = blockIdx.x;
    const int nq = H * maps, nk = G * maps;
    if (item >= nq + nk + G) return;
    float* buf = bufs[warp];
    const int ld = (nq + nk) * dim + G * vdim;
    const bool is_q = item < nq, is_k = !is_q && item < nq + nk;
    const int n = (is_q || is_k) ? dim : vdim;
    const int col = is_q ? item * dim : (is_k ? nq * dim + (item - nq) * dim : (nq + nk) * dim + (item - nq - nk) * vdim);
    const float* src = qkv + (size_t)t * ld + col;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) { const float v = src[i] + (bias ? bias[col + i] : 0.f); buf[i] = v; ss += v * v; }
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    if (w) {
        const float scale = rsqrtf(warp_sum(ss) / (float)n + eps);
        for (int i = lane; i < n; i += 32) buf[i] = buf[i] * scale * w[i];
    }
    __syncwarp();
    const int rd = (is_q || is_k) ? rdims : 0;
    const float* cs = cos_t + (size_t)t * (rd >> 1);
    const float* sn = sin_t + (size_t)t * (rd >> 1);
    T* dst;
    if (is_q) dst = q_out + (size_t)t * nq * dim + (size_t)item * dim;
    else {
        if (!store_kv) return;
        const int b = tok_seq[t], p = tok_pos[t];
        const size_t page = page_table[(size_t)b * table_width + p / QWB_MAPS_PAGE];
        if (is_k) {
            const int head = (item - nq) / maps, m = (item - nq) % maps;
            dst = k_pool + ((page * G + head) * QWB_MAPS_PAGE + p % QWB_MAPS_PAGE) * (size_t)(maps * dim) + m * dim;
        } else {
            dst = v_pool + ((page * G + (item - nq - nk)) * QWB_MAPS_PAGE + p % QWB_MAPS_PAGE) * (size_t)vdim;
        }
    }
    for (int i = lane; i < n; i += 32) dst[i] = from_f32<T>(rd > 0 ? maps_turned(buf, i, rd, cs, sn, interleaved) : buf[i]);
}

// `step`: 1 for the kernels that read value by value, 8 for those that copy 16 bytes at a time
static int check_maps_sizes(const char* what, int H, int G, int maps, int dim, int vdim, int table_width, int chunk, int step) {
    if (H <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", what, H, G);
    if (maps < 1 || maps > QWB_MAPS_MAX) return qwb_fail(QWB_ERR_ARG, "%s: %d score maps per head (1 or 2)", what, maps);
    if (dim <= 0 || dim % step || dim > QWB_MAPS_MAX_DIM || vdim <= 0 || vdim % step || vdim > QWB_MAPS_MAX_DIM)
        return qwb_fail(QWB_ERR_ARG, "%s: key size %d or value size %d is not a multiple of %d in [%d, %d]", what, dim, vdim, step, step, QWB_MAPS_MAX_DIM);
    if (table_width <= 0 || chunk < 0) return qwb_fail(QWB_ERR_ARG, "%s: bad table width %d or chunk %d", what, table_width, chunk);
    return 0;
}

extern "C" int qwb_maps_prep(const float* qkv, const float* bias, const float* qw, const float* kw, const float* cos_t, const float* sin_t,
                             const int* tok_seq, const int* tok_pos, const int* page_table, int table_width, void* q_out, void* k_pool,
                             void* v_pool, int dtype, int T, int H, int G, int maps, int dim, int vdim, int rdims, int interleaved,
                             float eps, int store_kv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (int rc = check_maps_sizes("maps_prep", H, G, maps, dim, vdim, table_width, 0, 1)) return rc;
    if (rdims < 0 || rdims > dim || rdims % 2) return qwb_fail(QWB_ERR_ARG, "maps_prep: a rotation of %d of %d values", rdims, dim);
    if (rdims > 0 && (!cos_t || !sin_t)) return qwb_fail(QWB_ERR_ARG, "maps_prep: a rotation without its table");
    dim3 grid(T, ((H + G) * maps + G + 3) / 4);
    if (dtype == QWB_DT_F32)
        qwb_launch(maps_prep_kernel<float>, grid, 128, 0, stream, qkv, bias, qw, kw, cos_t, sin_t, tok_seq, tok_pos, page_table, table_width,
                   (float*)q_out, (float*)k_pool, (float*)v_pool, H, G, maps, dim, vdim, rdims, interleaved, eps, store_kv);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(maps_prep_kernel<bf16>, grid, 128, 0, stream, qkv, bias, qw, kw, cos_t, sin_t, tok_seq, tok_pos, page_table, table_width,
                   (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, H, G, maps, dim, vdim, rdims, interleaved, eps, store_kv);
    else return qwb_fail(QWB_ERR_ARG, "maps_prep: unknown dtype %d", dtype);
    return qwb_check_launch("maps_prep");
}

// ---------------------------------------------------------------------------------
// prefill: one block per (tile of 16 queries, query head, sequence); 4 warps, each owns 4 queries; keys come in tiles of
// 32 (one key per lane), from the first key that the tile's first query sees to the tile's last query; the maps one
// after the other over the same tiles.
// ---------------------------------------------------------------------------------
template <typename T, int NC>   // NC = ceil(vdim / 32) rounded up to 2, 4 or 8
__global__ void maps_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                    const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                                    T* __restrict__ out, int H, int G, int maps, int dim, int vdim, int table_width, float scale,
                                    float softcap, int chunk, float lambda, int norm_out, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BQ = 16, BK = 32, QPW = 4, PG = QWB_MAPS_PAGE;
    extern __shared__ float smem[];
    float* Qs = smem;                         // [BQ][dim], already scaled
    float* Ks = Qs + BQ * dim;                // [BK][dim + 1]
    float* Vs = Ks + BK * (dim + 1);          // [BK][vdim]

    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    if (q0 >= n_new) return;
    const int g = h / (H / G);
    const int p0 = pos0[b];
    const int nq = min(BQ, n_new - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kdim = maps * dim;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

    float res[QPW][NC];                       // map 0's normed sums, then the difference
    const int k_last = p0 + q0 + nq - 1;
    const int k_first = maps_first_key(p0 + q0, chunk);
    const int* pages = page_table + (size_t)b * table_width;

    for (int mp = 0; mp < maps; ++mp) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < BQ * dim; idx += blockDim.x) {
            const int i = idx / dim, d = idx - i * dim;
            Qs[idx] = i < nq ? to_f32(q[((size_t)(t0 + q0 + i) * H + h) * kdim + mp * dim + d]) * scale : 0.f;
        }
        float m[QPW], l[QPW], acc[QPW][NC];
#pragma unroll
        for (int i = 0; i < QPW; ++i) {
            m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
        }
        for (int kt = (k_first / BK) * BK; kt <= k_last; kt += BK) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < BK * dim; idx += blockDim.x) {
                const int j = idx / dim, d = idx - j * dim, key = kt + j;
                Ks[j * (dim + 1) + d] = key <= k_last ? to_f32(k_pool[(((size_t)pages[key / PG] * G + g) * PG + key % PG) * kdim + mp * dim + d]) : 0.f;
            }
            for (int idx = threadIdx.x; idx < BK * vdim; idx += blockDim.x) {
                const int j = idx / vdim, d = idx - j * vdim, key = kt + j;
                Vs[idx] = key <= k_last ? to_f32(v_pool[(((size_t)pages[key / PG] * G + g) * PG + key % PG) * vdim + d]) : 0.f;
            }
            __syncthreads();

            float s[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) s[i] = 0.f;
            const float* krow = Ks + lane * (dim + 1);
            for (int d = 0; d < dim; ++d) {
                const float kd = krow[d];
#pragma unroll
                for (int i = 0; i < QPW; ++i) s[i] += Qs[(warp * QPW + i) * dim + d] * kd;
            }
            const int key = kt + lane;
            float p[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) {
                const int qi = warp * QPW + i;
                const int qp = p0 + q0 + qi;
                const bool ok = qi < nq && key <= qp && key >= maps_first_key(qp, chunk);
                const float si = ok ? maps_cap(s[i], softcap, inv_cap) : -INFINITY;
                const float m_new = fmaxf(m[i], warp_max(si));
                if (m_new == -INFINITY) { p[i] = 0.f; continue; }       // nothing visible so far (whole warp agrees)
                const float alpha = expf(m[i] - m_new);                 // m = -inf gives 0
                p[i] = ok ? expf(si - m_new) : 0.f;
                l[i] = l[i] * alpha + warp_sum(p[i]);
                m[i] = m_new;
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
            }
            for (int j = 0; j < BK; ++j) {
                float pj[QPW];
#pragma unroll
                for (int i = 0; i < QPW; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int d = lane + 32 * c;
                    if (d < vdim) {
                        const float v = Vs[j * vdim + d];
#pragma unroll
                        for (int i = 0; i < QPW; ++i) acc[i][c] += pj[i] * v;
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < QPW; ++i) {
            const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float a = acc[i][c] * inv;
                res[i][c] = mp == 0 ? a : res[i][c] - lambda * a;
            }
        }
    }

#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        float mul = 1.f;
        if (norm_out) {
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) if (lane + 32 * c < vdim) ss += res[i][c] * res[i][c];
            mul = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
        }
        if (qi >= nq) continue;
        T* o = out + ((size_t)(t0 + q0 + qi) * H + h) * vdim;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int d = lane + 32 * c;
            if (d < vdim) o[d] = from_f32<T>(res[i][c] * mul);
        }
    }
}

template <typename T>
static int launch_maps_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                               const int* pos0, void* out, int B, int max_new, int H, int G, int maps, int dim, int vdim, int table_width,
                               float scale, float softcap, int chunk, float lambda, int norm_out, float eps, float out_scale,
                               cudaStream_t stream) {
    const size_t smem = ((size_t)16 * dim + 32 * (dim + 1) + 32 * vdim) * sizeof(float);
    dim3 grid((max_new + 15) / 16, H, B);
    const int nc = (vdim + 31) / 32;
#define QWB_LAUNCH_MAPS_PREFILL(NC)                                                                              \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(maps_prefill_kernel<T, NC>,                                     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "maps_prefill: %s", cudaGetErrorString(e));      \
        }                                                                                                        \
        qwb_launch(maps_prefill_kernel<T, NC>, grid, 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, \
            page_table, cu_seqlens, pos0, (T*)out, H, G, maps, dim, vdim, table_width, scale, softcap, chunk, lambda, norm_out, \
            eps, out_scale);                                                                                     \
    } while (0)
    if (nc <= 2) QWB_LAUNCH_MAPS_PREFILL(2);
    else if (nc <= 4) QWB_LAUNCH_MAPS_PREFILL(4);
    else QWB_LAUNCH_MAPS_PREFILL(8);
#undef QWB_LAUNCH_MAPS_PREFILL
    return qwb_check_launch("maps_prefill");
}

// q [T, H, maps * dim]; out [T, H * vdim].
extern "C" int qwb_maps_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                                const int* pos0, void* out, int dtype, int B, int max_new, int H, int G, int maps, int dim, int vdim,
                                int table_width, float scale, float softcap, int chunk, float lambda, int norm_out, float eps,
                                float out_scale, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_maps_sizes("maps_prefill", H, G, maps, dim, vdim, table_width, chunk, 1)) return rc;
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "maps_prefill: batch %d or heads %d above 65535", B, H);
    if (dtype == QWB_DT_F32)
        return launch_maps_prefill<float>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, H, G, maps, dim, vdim, table_width,
                                          scale, softcap, chunk, lambda, norm_out, eps, out_scale, stream);
    if (dtype == QWB_DT_BF16)
        return launch_maps_prefill<bf16>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, H, G, maps, dim, vdim, table_width,
                                         scale, softcap, chunk, lambda, norm_out, eps, out_scale, stream);
    return qwb_fail(QWB_ERR_ARG, "maps_prefill: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// prefill on the tensor cores (bfloat16, mma.sync m16n8k16): block = 64 queries of one (sequence, query head), 4 warps of
// 16 rows; keys in tiles of 64 = one page of the cache, from the page of the first key that the tile's first query sees
// to the page of its last query.  The maps run one after the other over the same pages: map m reads columns
// [m * dim, (m + 1) * dim) of the key rows and the same values.  Q, K and V tiles sit in shared memory with rows padded
// by 16 bytes (conflict-free ldmatrix); K has two buffers, V one: the next tile's keys are copied in (cp.async) under
// this tile's work, its values under its own scores and softmax.  Scores, the cap, maxima, sums, accumulators, the
// difference of the maps and the norm are 32-bit; probabilities are rounded to bfloat16 for the second product.
// dim a multiple of 16, vdim of 8.
// ---------------------------------------------------------------------------------
#define MM_BQ 64
#define MM_BK 64
#define MM_PAD 8

__device__ __forceinline__ void mm_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mm_ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mm_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; `bytes` 0 writes zeros (src must still be a valid address)
__device__ __forceinline__ void mm_cp16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void mm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void mm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t mm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float mm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mm_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte pieces of a [rows][cpr pieces] tile, dealt to 128 threads in order: the thread's first piece and its stride,
// as (row, piece) pairs, so that the copy loops divide nothing
struct MmWalk {
    int r0, c0, dr, dc, cpr;
    __device__ __forceinline__ MmWalk(int tid, int pieces_per_row) : r0(tid / pieces_per_row), c0(tid % pieces_per_row),
        dr(128 / pieces_per_row), dc(128 % pieces_per_row), cpr(pieces_per_row) {}
    __device__ __forceinline__ void next(int& r, int& c) const { r += dr; c += dc; if (c >= cpr) { c -= cpr; ++r; } }
};

template <int NV, int MAPS>     // n-tiles of 8 value columns the accumulator has room for; score maps per head
__global__ void __launch_bounds__(128)
maps_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                        bf16* __restrict__ out, int H, int G, int dim, int vdim, int table_width, float scale, float softcap,
                        int chunk, float lambda, int norm_out, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int ldq = dim + MM_PAD, ldv = vdim + MM_PAD, kdim = MAPS * dim;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Kbuf = Qs + MM_BQ * ldq;                          // [2][64][ldq]
    bf16* Vbuf = Kbuf + 2 * MM_BK * ldq;                    // [64][ldv]

    // the last queries see the most keys: their blocks start first, so that the long blocks are not the launch's tail
    const int b = blockIdx.z, h = blockIdx.y, q0 = (int)(gridDim.x - 1 - blockIdx.x) * MM_BQ;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (q0 >= n) return;
    const int g_kv = h / (H / G);
    const int p0 = pos0[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = min(MM_BQ, n - q0);
    const int gr = lane >> 2, tq = lane & 3;
    const int pos_a = p0 + q0 + warp * 16 + gr, pos_b = pos_a + 8;  // positions of the thread's two rows
    const int lo_a = maps_first_key(pos_a, chunk), lo_b = maps_first_key(pos_b, chunk);

    const int k_hi = p0 + q0 + nq - 1;                              // last key any query of the tile sees
    const int k_lo = maps_first_key(p0 + q0, chunk);                // first key any of them sees
    const int nv_used = vdim / 8;
    const int first_page = k_lo / MM_BK, n_tiles = k_hi / MM_BK - first_page + 1;
    const int* pages = page_table + (size_t)b * table_width;
    const int warp_lo = p0 + q0 + warp * 16, warp_hi = warp_lo + 15;
    const int warp_first = maps_first_key(warp_hi, chunk);          // the first key that every row of the warp may see
    const float log2e = 1.4426950408889634f;
    // Scores in units of ln 2 (ex2 below).  With a cap c: c tanh(x / c) = c - 2 c / (e^(2 x / c) + 1), exact at both ends
    // (e^.. = inf or 0) and a few units of the last place in between: one ex2, one rcp and one fma a score.
    const float mul_s = softcap > 0.f ? scale / softcap * 2.f * log2e : scale * log2e;
    const float cap2 = softcap * log2e;
    const MmWalk walk_k(tid, dim / 8), walk_v(tid, vdim / 8);

    float res[MAPS > 1 ? NV : 1][4];                                // map 0's normed sums, until the difference is formed

#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        auto copy_keys = [&](int it, int stage) {                   // one commit group
            const int page = first_page + it;
            const int rows = min(MM_BK, k_hi + 1 - page * MM_BK);
            const bf16* ks = k_pool + ((size_t)pages[page] * G + g_kv) * MM_BK * kdim + mp * dim;
            bf16* Kd = Kbuf + stage * MM_BK * ldq;
            for (int r = walk_k.r0, c = walk_k.c0; r < MM_BK; walk_k.next(r, c))
                mm_cp16(Kd + r * ldq + c * 8, ks + (size_t)(r < rows ? r : 0) * kdim + c * 8, r < rows ? 16 : 0);
            mm_commit();
        };
        auto copy_values = [&](int it) {                            // one commit group
            const int page = first_page + it;
            const int rows = min(MM_BK, k_hi + 1 - page * MM_BK);
            const bf16* vs = v_pool + ((size_t)pages[page] * G + g_kv) * MM_BK * vdim;
            for (int r = walk_v.r0, c = walk_v.c0; r < MM_BK; walk_v.next(r, c))
                mm_cp16(Vbuf + r * ldv + c * 8, vs + (size_t)(r < rows ? r : 0) * vdim + c * 8, r < rows ? 16 : 0);
            mm_commit();
        };
        // this map's queries (the last readers of Qs, Kbuf and Vbuf passed the barrier that closed the map before)
        for (int r = walk_k.r0, c = walk_k.c0; r < MM_BQ; walk_k.next(r, c)) {
            const bool in = r < nq;
            mm_cp16(Qs + r * ldq + c * 8, q + ((size_t)(t0 + (in ? q0 + r : 0)) * H + h) * kdim + mp * dim + c * 8, in ? 16 : 0);
        }
        // groups in the order of their commits: [Q, K0], V0, K1, V1, K2, ...
        copy_keys(0, 0);
        copy_values(0);

        float o[NV][4];
#pragma unroll
        for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows gr and gr + 8 of the warp's 16

        for (int it = 0; it < n_tiles; ++it) {
            const bf16* Ks = Kbuf + (it & 1) * MM_BK * ldq;
            const bf16* Vs = Vbuf;
            const bool more = it + 1 < n_tiles;
            if (more) {                                             // the next keys into the other buffer (its last readers
                copy_keys(it + 1, (it + 1) & 1);                    // passed the barrier at the end of the round before)
                mm_wait<2>();                                       // this tile's keys (and Q) are there
            } else {
                mm_wait<1>();
            }
            __syncthreads();
            const int key0 = (first_page + it) * MM_BK;
            // a tile that no row of the warp sees (behind its last row, or before its chunk) is skipped by the warp
            const bool none = key0 > warp_hi || key0 + MM_BK <= maps_first_key(warp_lo, chunk);
            float s[8][4];
            if (!none) {
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
                for (int d = 0; d < dim; d += 16) {
                    uint32_t a0, a1, a2, a3;
                    mm_ldsm_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + d + (lane >> 4) * 8);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {                // two tiles of 8 keys a load
                        uint32_t b0, b1, b2, b3;
                        mm_ldsm_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane & 7) + (lane >> 4) * 8) * ldq + d + ((lane >> 3) & 1) * 8);
                        mm_mma(s[j], a0, a1, a2, a3, b0, b1);
                        mm_mma(s[j + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
                // a tile that every row of the warp sees whole needs no mask (most tiles of a long prompt)
                const bool whole = key0 + MM_BK - 1 <= warp_lo && key0 >= warp_first;
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        bool ok = true;
                        if (!whole) {
                            const int key = key0 + j * 8 + tq * 2 + (e & 1);
                            ok = key <= (e < 2 ? pos_a : pos_b) && key >= (e < 2 ? lo_a : lo_b) && key <= k_hi;
                        }
                        float v = s[j][e] * mul_s;
                        if (softcap > 0.f) v = fmaf(-2.f * cap2, mm_rcp(mm_ex2(v) + 1.f), cap2);
                        s[j][e] = ok ? v : -INFINITY;
                    }
                    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
                const float alpha0 = mm_ex2(m0 - base0), alpha1 = mm_ex2(m1 - base1);  // m = -inf gives 0
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    s[j][0] = mm_ex2(s[j][0] - base0); s[j][1] = mm_ex2(s[j][1] - base0);
                    s[j][2] = mm_ex2(s[j][2] - base1); s[j][3] = mm_ex2(s[j][3] - base1);
                    sum0 += s[j][0] + s[j][1];
                    sum1 += s[j][2] + s[j][3];
                }
                sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
                sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
                l0 = l0 * alpha0 + sum0; l1 = l1 * alpha1 + sum1;
                m0 = mn0; m1 = mn1;
#pragma unroll
                for (int j = 0; j < NV; ++j) { o[j][0] *= alpha0; o[j][1] *= alpha0; o[j][2] *= alpha1; o[j][3] *= alpha1; }
            }

            if (more) mm_wait<1>(); else mm_wait<0>();              // this tile's values are there
            __syncthreads();
            if (!none) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {                    // O += P V, 16 keys a step
                    const uint32_t a0 = mm_pack(s[2 * ks][0], s[2 * ks][1]), a1 = mm_pack(s[2 * ks][2], s[2 * ks][3]);
                    const uint32_t a2 = mm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = mm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                    for (int j = 0; j < NV; j += 2) {
                        if (j < nv_used) {                          // vdim / 8 may be odd: the second tile of a pair reads padding
                            uint32_t b0, b1, b2, b3;                // or the next row's start, and its result is never stored
                            mm_ldsm_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + j * 8 + (lane >> 4) * 8);
                            mm_mma(o[j], a0, a1, a2, a3, b0, b1);
                            if (j + 1 < NV) mm_mma(o[j + 1], a0, a1, a2, a3, b2, b3);
                        }
                    }
                }
            }
            __syncthreads();                                        // the values' buffer may be copied into again
            if (more) copy_values(it + 1);
        }

        const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
        if (MAPS > 1 && mp == 0) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                res[MAPS > 1 ? j : 0][0] = o[j][0] * inv0; res[MAPS > 1 ? j : 0][1] = o[j][1] * inv0;
                res[MAPS > 1 ? j : 0][2] = o[j][2] * inv1; res[MAPS > 1 ? j : 0][3] = o[j][3] * inv1;
            }
        } else {
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                o[j][0] *= inv0; o[j][1] *= inv0; o[j][2] *= inv1; o[j][3] *= inv1;
                if (MAPS > 1) {
                    o[j][0] = res[MAPS > 1 ? j : 0][0] - lambda * o[j][0]; o[j][1] = res[MAPS > 1 ? j : 0][1] - lambda * o[j][1];
                    o[j][2] = res[MAPS > 1 ? j : 0][2] - lambda * o[j][2]; o[j][3] = res[MAPS > 1 ? j : 0][3] - lambda * o[j][3];
                }
                if (j < nv_used) { ss0 += o[j][0] * o[j][0] + o[j][1] * o[j][1]; ss1 += o[j][2] * o[j][2] + o[j][3] * o[j][3]; }
            }
            float mul0 = 1.f, mul1 = 1.f;
            if (norm_out) {
                ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
                ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
                mul0 = rsqrtf(ss0 / (float)vdim + eps) * out_scale;
                mul1 = rsqrtf(ss1 / (float)vdim + eps) * out_scale;
            }
            const int row_a = warp * 16 + gr, row_b = row_a + 8;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (j < nv_used) {
                    const int col = j * 8 + tq * 2;
                    if (row_a < nq) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + q0 + row_a) * H + h) * vdim + col) = mm_pack(o[j][0] * mul0, o[j][1] * mul0);
                    if (row_b < nq) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + q0 + row_b) * H + h) * vdim + col) = mm_pack(o[j][2] * mul1, o[j][3] * mul1);
                }
            }
        }
    }
}

// Two maps in ONE pass over the keys (values of up to 128): a tile's key rows hold both maps side by side, as the cache
// has them, and so do the query rows; a warp forms map 0's scores and probabilities, then map 1's, and both products
// with the values read each value fragment once.  Twice the accumulators (128 registers at values of 128), half the
// tiles, copies and barriers of the kernel above, and no result of the first map to keep.
template <int NV>
__global__ void __launch_bounds__(128)
maps_prefill_mma_pair_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                             const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                             bf16* __restrict__ out, int H, int G, int dim, int vdim, int table_width, float scale, float softcap,
                             int chunk, float lambda, int norm_out, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int kdim = 2 * dim, ldq = kdim + MM_PAD, ldv = vdim + MM_PAD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Kbuf = Qs + MM_BQ * ldq;                          // [2][64][ldq]
    bf16* Vbuf = Kbuf + 2 * MM_BK * ldq;                    // [64][ldv]

    const int b = blockIdx.z, h = blockIdx.y, q0 = (int)(gridDim.x - 1 - blockIdx.x) * MM_BQ;   // long blocks first
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (q0 >= n) return;
    const int g_kv = h / (H / G);
    const int p0 = pos0[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = min(MM_BQ, n - q0);
    const int gr = lane >> 2, tq = lane & 3;
    const int pos_a = p0 + q0 + warp * 16 + gr, pos_b = pos_a + 8;
    const int lo_a = maps_first_key(pos_a, chunk), lo_b = maps_first_key(pos_b, chunk);
    const int k_hi = p0 + q0 + nq - 1, k_lo = maps_first_key(p0 + q0, chunk);
    const int nv_used = vdim / 8;
    const int first_page = k_lo / MM_BK, n_tiles = k_hi / MM_BK - first_page + 1;
    const int* pages = page_table + (size_t)b * table_width;
    const int warp_lo = p0 + q0 + warp * 16, warp_hi = warp_lo + 15;
    const int warp_first = maps_first_key(warp_hi, chunk);
    const float log2e = 1.4426950408889634f;
    const float mul_s = softcap > 0.f ? scale / softcap * 2.f * log2e : scale * log2e;
    const float cap2 = softcap * log2e;
    const MmWalk walk_k(tid, kdim / 8), walk_v(tid, vdim / 8);

    auto copy_keys = [&](int it, int stage) {
        const int page = first_page + it;
        const int rows = min(MM_BK, k_hi + 1 - page * MM_BK);
        const bf16* ks = k_pool + ((size_t)pages[page] * G + g_kv) * MM_BK * kdim;
        bf16* Kd = Kbuf + stage * MM_BK * ldq;
        for (int r = walk_k.r0, c = walk_k.c0; r < MM_BK; walk_k.next(r, c))
            mm_cp16(Kd + r * ldq + c * 8, ks + (size_t)(r < rows ? r : 0) * kdim + c * 8, r < rows ? 16 : 0);
        mm_commit();
    };
    auto copy_values = [&](int it) {
        const int page = first_page + it;
        const int rows = min(MM_BK, k_hi + 1 - page * MM_BK);
        const bf16* vs = v_pool + ((size_t)pages[page] * G + g_kv) * MM_BK * vdim;
        for (int r = walk_v.r0, c = walk_v.c0; r < MM_BK; walk_v.next(r, c))
            mm_cp16(Vbuf + r * ldv + c * 8, vs + (size_t)(r < rows ? r : 0) * vdim + c * 8, r < rows ? 16 : 0);
        mm_commit();
    };
    for (int r = walk_k.r0, c = walk_k.c0; r < MM_BQ; walk_k.next(r, c)) {
        const bool in = r < nq;
        mm_cp16(Qs + r * ldq + c * 8, q + ((size_t)(t0 + (in ? q0 + r : 0)) * H + h) * kdim + c * 8, in ? 16 : 0);
    }
    copy_keys(0, 0);
    copy_values(0);

    float o[2][NV][4];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
#pragma unroll
        for (int j = 0; j < NV; ++j) o[mp][j][0] = o[mp][j][1] = o[mp][j][2] = o[mp][j][3] = 0.f;
    float m0[2] = {-INFINITY, -INFINITY}, m1[2] = {-INFINITY, -INFINITY}, l0[2] = {0.f, 0.f}, l1[2] = {0.f, 0.f};

    for (int it = 0; it < n_tiles; ++it) {
        const bf16* Ks = Kbuf + (it & 1) * MM_BK * ldq;
        const bf16* Vs = Vbuf;
        const bool more = it + 1 < n_tiles;
        if (more) { copy_keys(it + 1, (it + 1) & 1); mm_wait<2>(); } else { mm_wait<1>(); }
        __syncthreads();
        const int key0 = (first_page + it) * MM_BK;
        const bool none = key0 > warp_hi || key0 + MM_BK <= maps_first_key(warp_lo, chunk);
        const bool whole = key0 + MM_BK - 1 <= warp_lo && key0 >= warp_first;
        uint32_t pk[2][4][4];                                       // both maps' probabilities as the second product's A operands
        if (!none) {
#pragma unroll
            for (int mp = 0; mp < 2; ++mp) {
                float s[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
                for (int d = mp * dim; d < (mp + 1) * dim; d += 16) {
                    uint32_t a0, a1, a2, a3;
                    mm_ldsm_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + d + (lane >> 4) * 8);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        uint32_t b0, b1, b2, b3;
                        mm_ldsm_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane & 7) + (lane >> 4) * 8) * ldq + d + ((lane >> 3) & 1) * 8);
                        mm_mma(s[j], a0, a1, a2, a3, b0, b1);
                        mm_mma(s[j + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        bool ok = true;
                        if (!whole) {
                            const int key = key0 + j * 8 + tq * 2 + (e & 1);
                            ok = key <= (e < 2 ? pos_a : pos_b) && key >= (e < 2 ? lo_a : lo_b) && key <= k_hi;
                        }
                        float v = s[j][e] * mul_s;
                        if (softcap > 0.f) v = fmaf(-2.f * cap2, mm_rcp(mm_ex2(v) + 1.f), cap2);
                        s[j][e] = ok ? v : -INFINITY;
                    }
                    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0[mp], mx0), mn1 = fmaxf(m1[mp], mx1);
                const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
                const float alpha0 = mm_ex2(m0[mp] - base0), alpha1 = mm_ex2(m1[mp] - base1);
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    s[j][0] = mm_ex2(s[j][0] - base0); s[j][1] = mm_ex2(s[j][1] - base0);
                    s[j][2] = mm_ex2(s[j][2] - base1); s[j][3] = mm_ex2(s[j][3] - base1);
                    sum0 += s[j][0] + s[j][1];
                    sum1 += s[j][2] + s[j][3];
                }
                sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
                sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
                l0[mp] = l0[mp] * alpha0 + sum0; l1[mp] = l1[mp] * alpha1 + sum1;
                m0[mp] = mn0; m1[mp] = mn1;
#pragma unroll
                for (int j = 0; j < NV; ++j) { o[mp][j][0] *= alpha0; o[mp][j][1] *= alpha0; o[mp][j][2] *= alpha1; o[mp][j][3] *= alpha1; }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    pk[mp][ks][0] = mm_pack(s[2 * ks][0], s[2 * ks][1]); pk[mp][ks][1] = mm_pack(s[2 * ks][2], s[2 * ks][3]);
                    pk[mp][ks][2] = mm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]); pk[mp][ks][3] = mm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
                }
            }
        }
        if (more) mm_wait<1>(); else mm_wait<0>();                  // this tile's values are there
        __syncthreads();
        if (!none) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int j = 0; j < NV; j += 2) {
                    if (j < nv_used) {
                        uint32_t b0, b1, b2, b3;
                        mm_ldsm_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + j * 8 + (lane >> 4) * 8);
#pragma unroll
                        for (int mp = 0; mp < 2; ++mp) {
                            mm_mma(o[mp][j], pk[mp][ks][0], pk[mp][ks][1], pk[mp][ks][2], pk[mp][ks][3], b0, b1);
                            if (j + 1 < NV) mm_mma(o[mp][j + 1], pk[mp][ks][0], pk[mp][ks][1], pk[mp][ks][2], pk[mp][ks][3], b2, b3);
                        }
                    }
                }
            }
        }
        __syncthreads();
        if (more) copy_values(it + 1);
    }

    const float ia0 = l0[0] > 0.f ? 1.f / l0[0] : 0.f, ia1 = l1[0] > 0.f ? 1.f / l1[0] : 0.f;
    const float ib0 = l0[1] > 0.f ? lambda / l0[1] : 0.f, ib1 = l1[1] > 0.f ? lambda / l1[1] : 0.f;
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        o[0][j][0] = o[0][j][0] * ia0 - o[1][j][0] * ib0; o[0][j][1] = o[0][j][1] * ia0 - o[1][j][1] * ib0;
        o[0][j][2] = o[0][j][2] * ia1 - o[1][j][2] * ib1; o[0][j][3] = o[0][j][3] * ia1 - o[1][j][3] * ib1;
        if (j < nv_used) { ss0 += o[0][j][0] * o[0][j][0] + o[0][j][1] * o[0][j][1]; ss1 += o[0][j][2] * o[0][j][2] + o[0][j][3] * o[0][j][3]; }
    }
    float mul0 = 1.f, mul1 = 1.f;
    if (norm_out) {
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
        mul0 = rsqrtf(ss0 / (float)vdim + eps) * out_scale;
        mul1 = rsqrtf(ss1 / (float)vdim + eps) * out_scale;
    }
    const int row_a = warp * 16 + gr, row_b = row_a + 8;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        if (j < nv_used) {
            const int col = j * 8 + tq * 2;
            if (row_a < nq) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + q0 + row_a) * H + h) * vdim + col) = mm_pack(o[0][j][0] * mul0, o[0][j][1] * mul0);
            if (row_b < nq) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + q0 + row_b) * H + h) * vdim + col) = mm_pack(o[0][j][2] * mul1, o[0][j][3] * mul1);
        }
    }
}

// Q and two key buffers [64][dim + 8] and one value buffer [64][vdim + 8] of bfloat16
static size_t mm_smem_bytes(int dim, int vdim) {
    return ((size_t)3 * MM_BK * (dim + MM_PAD) + (size_t)MM_BK * (vdim + MM_PAD)) * sizeof(bf16);
}

extern "C" int qwb_maps_prefill_mma_fits(int dtype, int maps, int dim, int vdim) {
    return dtype == QWB_DT_BF16 && maps >= 1 && maps <= QWB_MAPS_MAX && dim > 0 && dim % 16 == 0 && vdim > 0 && vdim % 8 == 0 &&
           dim <= QWB_MAPS_MAX_DIM && vdim <= QWB_MAPS_MAX_DIM && mm_smem_bytes(dim, vdim) <= 220 * 1024;
}

// q [T, H, maps * dim] bfloat16; out [T, H * vdim] bfloat16.
extern "C" int qwb_maps_prefill_mma(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                                    const int* pos0, void* out, int B, int max_new, int H, int G, int maps, int dim, int vdim,
                                    int table_width, float scale, float softcap, int chunk, float lambda, int norm_out, float eps,
                                    float out_scale, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_maps_sizes("maps_prefill_mma", H, G, maps, dim, vdim, table_width, chunk, 8)) return rc;
    if (!qwb_maps_prefill_mma_fits(QWB_DT_BF16, maps, dim, vdim))
        return qwb_fail(QWB_ERR_ARG, "maps_prefill_mma: keys of %d (a multiple of 16) and values of %d (of 8) that fit in shared memory", dim, vdim);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "maps_prefill_mma: batch %d or heads %d above 65535", B, H);
    for (const void* p : {q, k_pool, v_pool, (const void*)out})
        if ((uintptr_t)p % 16) return qwb_fail(QWB_ERR_ARG, "maps_prefill_mma: a tensor is not 16-byte aligned");
    const size_t smem = mm_smem_bytes(dim, vdim);
    const dim3 grid((max_new + MM_BQ - 1) / MM_BQ, H, B);
#define QWB_MM(NV, MAPS)                                                                                                        \
    do {                                                                                                                        \
        if (smem > 48 * 1024) {                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(maps_prefill_mma_kernel<NV, MAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "maps_prefill_mma: %s", cudaGetErrorString(e));                 \
        }                                                                                                                       \
        qwb_launch(maps_prefill_mma_kernel<NV, MAPS>, grid, 128, smem, stream, (const bf16*)q, (const bf16*)k_pool,             \
                   (const bf16*)v_pool, page_table, cu_seqlens, pos0, (bf16*)out, H, G, dim, vdim, table_width, scale, softcap, \
                   chunk, lambda, norm_out, eps, out_scale);                                                                    \
    } while (0)
#define QWB_MM_SIZES(MAPS)                                                                                                      \
    do {                                                                                                                        \
        if (vdim <= 32) QWB_MM(4, MAPS); else if (vdim <= 64) QWB_MM(8, MAPS); else if (vdim <= 128) QWB_MM(16, MAPS);          \
        else QWB_MM(32, MAPS);                                                                                                  \
    } while (0)
    const size_t smem_pair = mm_smem_bytes(2 * dim, vdim);
    if (maps == 2 && vdim <= 128 && smem_pair <= 220 * 1024) {         // both maps in one pass
#define QWB_MM_PAIR(NV)                                                                                                         \
    do {                                                                                                                        \
        if (smem_pair > 48 * 1024) {                                                                                            \
            cudaError_t e = cudaFuncSetAttribute(maps_prefill_mma_pair_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_pair); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "maps_prefill_mma: %s", cudaGetErrorString(e));                 \
        }                                                                                                                       \
        qwb_launch(maps_prefill_mma_pair_kernel<NV>, grid, 128, smem_pair, stream, (const bf16*)q, (const bf16*)k_pool,         \
                   (const bf16*)v_pool, page_table, cu_seqlens, pos0, (bf16*)out, H, G, dim, vdim, table_width, scale, softcap, \
                   chunk, lambda, norm_out, eps, out_scale);                                                                    \
    } while (0)
        if (vdim <= 32) QWB_MM_PAIR(4); else if (vdim <= 64) QWB_MM_PAIR(8); else QWB_MM_PAIR(16);
#undef QWB_MM_PAIR
    } else if (maps == 1) QWB_MM_SIZES(1); else QWB_MM_SIZES(2);
#undef QWB_MM_SIZES
#undef QWB_MM
    return qwb_check_launch("maps_prefill_mma");
}

// ---------------------------------------------------------------------------------
// decode: one new token per sequence (its position is len - 1).  The keys it sees, first .. len - 1 with first the start
// of its chunk (or 0), are cut into runs of whole pages counted from the page of the first key: 2 pages a run, doubled
// while that would give more than 64 runs.  Which keys a run holds follows from the sequence's own length alone.
// Block = (run, key/value head and slice of its rows, sequence), 128 threads; a row is a (query head, map) pair, up to 8 a
// block: a page's K and V tiles go to shared memory; thread (key, half of the rows) forms the scores; a warp per row
// updates maximum and sum; thread d accumulates p v for all rows.
// ---------------------------------------------------------------------------------
__device__ __host__ __forceinline__ int maps_run_pages(int first_key, int len) {
    const int span = (len - 1) / QWB_MAPS_PAGE - first_key / QWB_MAPS_PAGE + 1;
    int rp = QWB_MAPS_RUN_PAGES;
    while (span > rp * QWB_MAPS_MAX_RUNS) rp *= 2;
    return rp;
}

__device__ __forceinline__ void maps_cp16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}

template <typename T>
__global__ void maps_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                   const int* __restrict__ page_table, const int* __restrict__ seq_len, float* __restrict__ part_acc,
                                   float* __restrict__ part_m, float* __restrict__ part_l, int H, int G, int maps, int dim, int vdim,
                                   int table_width, float scale, float softcap, int chunk, int n_runs) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int RT = QWB_MAPS_ROWS, VEC = Vec16<T>::N, PG = QWB_MAPS_PAGE;
    const int b = blockIdx.z, run = blockIdx.x;
    const int len = seq_len[b];
    const int first = maps_first_key(len - 1, chunk);
    const int rp = maps_run_pages(first, len);
    const int page_lo = first / PG;
    const int row_first = max(first, (page_lo + run * rp) * PG);
    const int row_end = min(len, (page_lo + (run + 1) * rp) * PG);
    if (row_first >= row_end) return;

    const int QG = H / G, rows_g = QG * maps, slices = (rows_g + RT - 1) / RT;
    const int g = blockIdx.y / slices, r0 = (blockIdx.y % slices) * RT;       // rows of this key/value head: head-in-group * maps + map
    const int rcount = min(RT, rows_g - r0);
    const int kdim = maps * dim;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kld = kdim + VEC;                         // a key row and 16 bytes: rows start in different banks
    T* Kt = reinterpret_cast<T*>(smem_raw);             // [PG][kdim + VEC]
    T* Vt = Kt + (size_t)PG * kld;                      // [PG][vdim]
    float* qs = reinterpret_cast<float*>(Vt + (size_t)PG * vdim);   // [RT][dim], scaled
    float* sc = qs + RT * dim;                          // [RT][PG]
    float* m_s = sc + RT * PG;                          // [RT]
    float* l_s = m_s + RT;
    float* a_s = l_s + RT;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // row r0 + ri of head g: query head g * QG + (r0 + ri) / maps, map (r0 + ri) % maps; q is [B, H, maps * dim], so the
    // rows of a key/value head lie one after the other
    const T* qrow = q + ((size_t)b * H + (size_t)g * QG) * kdim + (size_t)r0 * dim;
    for (int idx = tid; idx < RT * dim; idx += blockDim.x) {
        const int ri = idx / dim;
        qs[idx] = ri < rcount ? to_f32(qrow[idx]) * scale : 0.f;
    }
    if (tid < RT) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f; }

    float acc[RT][2];
#pragma unroll
    for (int ri = 0; ri < RT; ++ri) acc[ri][0] = acc[ri][1] = 0.f;

    const int* pages = page_table + (size_t)b * table_width;
    const int my_key = tid % PG, my_slice = tid / PG;                 // two threads a key; each takes every second row
    const int nchunk = kdim / VEC, dchunk = dim / VEC;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

    for (int base = (row_first / PG) * PG; base < row_end; base += PG) {
        const int n_keys = min(PG, row_end - base);
        const size_t tile = (size_t)pages[base / PG] * G + g;
        __syncthreads();                                              // the last page's tiles are no longer read
        {
            const uint4* ksrc = reinterpret_cast<const uint4*>(k_pool + tile * PG * kdim);
            const uint4* vsrc = reinterpret_cast<const uint4*>(v_pool + tile * PG * vdim);
            uint4* kdst = reinterpret_cast<uint4*>(Kt);
            uint4* vdst = reinterpret_cast<uint4*>(Vt);
            for (int i = tid; i < n_keys * nchunk; i += blockDim.x) maps_cp16(kdst + i + i / nchunk, ksrc + i);     // row r starts at r * (nchunk + 1)
            asm volatile("cp.async.commit_group;" ::: "memory");
            for (int i = tid; i < n_keys * vdim / VEC; i += blockDim.x) maps_cp16(vdst + i, vsrc + i);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");     // the keys are there; the values arrive under the scores
        }
        __syncthreads();

        if (my_key < n_keys) {
            const Vec16<T>* krow = reinterpret_cast<const Vec16<T>*>(Kt + (size_t)my_key * kld);
            const bool ok = base + my_key >= row_first;
            // rows my_slice, my_slice + 2, ... of the block: r0 and the stride are even, so with one or two maps they all
            // belong to one map, and a piece of the key is read once for all of them
            const int mp = (r0 + my_slice) % maps;
            float s[RT / 2];
#pragma unroll
            for (int k = 0; k < RT / 2; ++k) s[k] = 0.f;
            for (int ch = 0; ch < dchunk; ++ch) {
                float kf[VEC];
                krow[mp * dchunk + ch].get(kf);
#pragma unroll
                for (int k = 0; k < RT / 2; ++k) {                  // rows past rcount hold zeros
                    const float4* qr = reinterpret_cast<const float4*>(qs + (my_slice + 2 * k) * dim + ch * VEC);
#pragma unroll
                    for (int e = 0; e < VEC / 4; ++e) {
                        const float4 qv = qr[e];
                        s[k] += qv.x * kf[4 * e] + qv.y * kf[4 * e + 1] + qv.z * kf[4 * e + 2] + qv.w * kf[4 * e + 3];
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < RT / 2; ++k) {
                const int ri = my_slice + 2 * k;
                if (ri < rcount) sc[ri * PG + my_key] = ok ? maps_cap(s[k], softcap, inv_cap) : -INFINITY;
            }
        }
        __syncthreads();

        for (int ri = warp; ri < rcount; ri += (blockDim.x >> 5)) {
            float mx = -INFINITY;
            for (int j = lane; j < n_keys; j += 32) mx = fmaxf(mx, sc[ri * PG + j]);
            mx = warp_max(mx);
            const float m_old = m_s[ri], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < n_keys; j += 32) {
                const float sj = sc[ri * PG + j];
                const float pj = (m_new == -INFINITY || sj == -INFINITY) ? 0.f : expf(sj - m_new);
                sc[ri * PG + j] = pj;
                sum += pj;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
                a_s[ri] = alpha;
                l_s[ri] = l_s[ri] * alpha + sum;
                m_s[ri] = m_new;
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * 128;
            if (d < vdim) {
#pragma unroll
                for (int ri = 0; ri < RT; ++ri) if (ri < rcount) acc[ri][c] *= a_s[ri];
                int j = 0;
                for (; j + 4 <= n_keys; j += 4) {                    // four keys' weights of a row in one load
                    const float v0 = to_f32(Vt[(size_t)j * vdim + d]), v1 = to_f32(Vt[(size_t)(j + 1) * vdim + d]);
                    const float v2 = to_f32(Vt[(size_t)(j + 2) * vdim + d]), v3 = to_f32(Vt[(size_t)(j + 3) * vdim + d]);
#pragma unroll
                    for (int ri = 0; ri < RT; ++ri)
                        if (ri < rcount) {
                            const float4 p = *reinterpret_cast<const float4*>(sc + ri * PG + j);
                            acc[ri][c] += p.x * v0 + p.y * v1 + p.z * v2 + p.w * v3;
                        }
                }
                for (; j < n_keys; ++j) {
                    const float v = to_f32(Vt[(size_t)j * vdim + d]);
#pragma unroll
                    for (int ri = 0; ri < RT; ++ri) if (ri < rcount) acc[ri][c] += sc[ri * PG + j] * v;
                }
            }
        }
    }
    __syncthreads();

    const size_t row_base = ((size_t)b * G + g) * rows_g + r0;        // rows of all heads: [B, H * maps]
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = tid + c * 128;
        if (d >= vdim) continue;
#pragma unroll
        for (int ri = 0; ri < RT; ++ri)
            if (ri < rcount) part_acc[((row_base + ri) * n_runs + run) * vdim + d] = acc[ri][c];
    }
    if (tid < rcount) {
        const size_t at = (row_base + tid) * n_runs + run;
        part_m[at] = m_s[tid];
        part_l[at] = l_s[tid];
    }
}

// Per (query head, sequence): each map's a = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M), M = max_r m_r, over the
// sequence's runs in index order; then the difference of the maps, the norm and the factor.  grid (H, B), 128 threads:
// warp m first makes map m's weights e^(m_r - M) / L once for all columns, then thread d sums its column.
template <typename T>
__global__ void maps_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m, const float* __restrict__ part_l,
                                  const int* __restrict__ seq_len, T* __restrict__ out, int H, int maps, int vdim, int chunk, int n_runs,
                                  float lambda, int norm_out, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[32];
    __shared__ float wts[QWB_MAPS_MAX][QWB_MAPS_MAX_RUNS];
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int len = seq_len[b];
    const int first = maps_first_key(len - 1, chunk);
    const int rp = maps_run_pages(first, len);
    const int runs = min(n_runs, ((len - 1) / QWB_MAPS_PAGE - first / QWB_MAPS_PAGE) / rp + 1);
    if (warp < maps) {
        const size_t row = ((size_t)b * H + h) * maps + warp;
        float M = -INFINITY;
        for (int r = lane; r < runs; r += 32) M = fmaxf(M, part_m[row * n_runs + r]);
        M = warp_max(M);
        float L = 0.f;
        for (int r = lane; r < runs; r += 32) {
            const float e = M == -INFINITY ? 0.f : expf(part_m[row * n_runs + r] - M);
            wts[warp][r] = e;
            L += part_l[row * n_runs + r] * e;
        }
        L = warp_sum(L);
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int r = lane; r < runs; r += 32) wts[warp][r] *= inv;
    }
    __syncthreads();
    float res[2] = {0.f, 0.f};
    for (int mp = 0; mp < maps; ++mp) {
        const size_t row = ((size_t)b * H + h) * maps + mp;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * 128;
            if (d >= vdim) continue;
            const float* col = part_acc + row * n_runs * vdim + d;
            float a = 0.f;
#pragma unroll 8
            for (int r = 0; r < runs; ++r) a += col[(size_t)r * vdim] * wts[mp][r];
            res[c] = mp == 0 ? a : res[c] - lambda * a;
        }
    }
    float mul = 1.f;
    if (norm_out) {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) if (tid + c * 128 < vdim) ss += res[c] * res[c];
        mul = rsqrtf(block_sum(ss, red) / (float)vdim + eps) * out_scale;
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = tid + c * 128;
        if (d < vdim) out[((size_t)b * H + h) * vdim + d] = from_f32<T>(res[c] * mul);
    }
}

// runs of the grid for sequences of up to max_len tokens
extern "C" int qwb_maps_decode_runs(int max_len, int chunk) {
    if (max_len <= 0) return 1;
    // the most pages a sequence's visible keys touch: a chunk may begin anywhere in its first page
    const int pages_all = (max_len + QWB_MAPS_PAGE - 1) / QWB_MAPS_PAGE;
    const int pages = chunk > 0 ? min(pages_all, (chunk + QWB_MAPS_PAGE - 2) / QWB_MAPS_PAGE + 1) : pages_all;
    const int runs = (pages + QWB_MAPS_RUN_PAGES - 1) / QWB_MAPS_RUN_PAGES;
    return runs < QWB_MAPS_MAX_RUNS ? runs : QWB_MAPS_MAX_RUNS;
}

extern "C" long long qwb_maps_decode_scratch_floats(int B, int H, int maps, int vdim, int n_runs) {
    return (long long)B * H * maps * n_runs * (vdim + 2);
}

template <typename T>
static int launch_maps_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                              float* scratch, void* out, int B, int H, int G, int maps, int dim, int vdim, int table_width, float scale,
                              float softcap, int chunk, int n_runs, float lambda, int norm_out, float eps, float out_scale,
                              cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    const int kdim = maps * dim;
    const size_t rows = (size_t)B * H * maps;
    float* part_acc = scratch;
    float* part_m = part_acc + rows * n_runs * vdim;
    float* part_l = part_m + rows * n_runs;
    const size_t smem = ((size_t)QWB_MAPS_PAGE * (kdim + VEC) + (size_t)QWB_MAPS_PAGE * vdim) * sizeof(T) +
                        ((size_t)QWB_MAPS_ROWS * dim + QWB_MAPS_ROWS * QWB_MAPS_PAGE + 3 * QWB_MAPS_ROWS) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(maps_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "maps_decode: %s", cudaGetErrorString(e));
    }
    const int rows_g = (H / G) * maps, slices = (rows_g + QWB_MAPS_ROWS - 1) / QWB_MAPS_ROWS;
    qwb_launch(maps_decode_kernel<T>, dim3(n_runs, G * slices, B), 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool,
               page_table, seq_len, part_acc, part_m, part_l, H, G, maps, dim, vdim, table_width, scale, softcap, chunk, n_runs);
    if (int rc = qwb_check_launch("maps_decode")) return rc;
    qwb_launch(maps_merge_kernel<T>, dim3(H, B), 128, 0, stream, (const float*)part_acc, (const float*)part_m, (const float*)part_l,
               seq_len, (T*)out, H, maps, vdim, chunk, n_runs, lambda, norm_out, eps, out_scale);
    return qwb_check_launch("maps_merge");
}

// q [B, H, maps * dim]; out [B, H * vdim]; scratch: qwb_maps_decode_scratch_floats floats.
extern "C" int qwb_maps_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                               float* scratch, void* out, int dtype, int B, int H, int G, int maps, int dim, int vdim, int table_width,
                               float scale, float softcap, int chunk, int n_runs, float lambda, int norm_out, float eps, float out_scale,
                               cudaStream_t stream) {
    if (B <= 0) return 0;
    if (int rc = check_maps_sizes("maps_decode", H, G, maps, dim, vdim, table_width, chunk, 8)) return rc;
    if (n_runs <= 0 || n_runs > 65535 || B > 65535) return qwb_fail(QWB_ERR_ARG, "maps_decode: %d runs, %d sequences", n_runs, B);
    if (dtype == QWB_DT_F32)
        return launch_maps_decode<float>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, H, G, maps, dim, vdim, table_width, scale,
                                         softcap, chunk, n_runs, lambda, norm_out, eps, out_scale, stream);
    if (dtype == QWB_DT_BF16)
        return launch_maps_decode<bf16>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, H, G, maps, dim, vdim, table_width, scale,
                                        softcap, chunk, n_runs, lambda, norm_out, eps, out_scale, stream);
    return qwb_fail(QWB_ERR_ARG, "maps_decode: unknown dtype %d", dtype);
}
