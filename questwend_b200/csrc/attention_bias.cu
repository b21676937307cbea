// Softmax attention over the paged cache whose scores are shaped head by head, and whose heads may be mixed after the
// softmax.  Query head h reads key head g = h / (H / G); everything below is optional and a parameter:
//   score = q . k * scale * head_scale[h]                     (a learned number per head)
//   softcap > 0:  score <- softcap * tanh(score / softcap)
//   slopes:       score <- score - slopes[h] * (p - j)        (a bias that grows with the distance of key j from query p)
//   mask:         key j is seen from position p when j <= p and (window > 0) p - j < window
//   sinks:        the softmax's denominator also holds exp(sinks[h]): a key without a value
//   all_values:   head h's weights are applied to the values of EVERY value head c, out [T, H, G, vdim]; the mix of the
//                 heads' weights after the softmax, w'_h = sum_g M[h, g] w_g, is linear in the weights, so head h's output
//                 is sum_g M[h, g] * (w_g applied to the values of h's own value head), which bias_head_mix forms
//   gate:         a head's output times sigmoid(gate[t, h])
// Scores, maxima, sums and accumulators are 32-bit; q and the cache are float or bfloat16.
// The cache: K pool [pages, G, 64, dim], V pool [pages, G, 64, vdim].
//
//   bias_prep      bias, per-head RMS norm of q and k (a weight of dim values shared by the heads), rotation of the first
//                  rdims values of every head of q and k, cache write of a step's tokens (the values may be the keys as
//                  projected, before norm and rotation); q out
//   bias_prefill   any number of new tokens per sequence (float and bfloat16, any sizes up to 256)
//   bias_prefill_mma  bfloat16 prompts on the tensor cores
//   bias_decode    one new token per sequence: runs of pages, one block of threads a run, then bias_merge, which also adds
//                  the sink
//   bias_head_mix  the mix of the heads and the gate
//   bias_decode_mixed  one new token per sequence with mixed heads, in two passes over the keys
#include "common.cuh"

#define QWB_BIAS_MAX_DIM 256
#define QWB_BIAS_PAGE 64
#define QWB_BIAS_ROWS 8           // query heads per block of the decode kernel
#define QWB_BIAS_RUN_PAGES 2      // pages per run of the decode kernel, doubled while a sequence would have more than ...
#define QWB_BIAS_MAX_RUNS 64      // ... this many runs: follows from the sequence's own length, not from the batch

// value i of a vector after its first n values were turned by the angle whose cos and sin are cs[m], sn[m] for pair m
__device__ __forceinline__ float bias_turned(const float* v, int i, int n, const float* cs, const float* sn, int interleaved) {
    if (i >= n) return v[i];
    const int half = n >> 1;
    int m, first;
    float a, b;
    if (interleaved) { m = i >> 1; first = !(i & 1); a = v[2 * m]; b = v[2 * m + 1]; }
    else { m = i < half ? i : i - half; first = i < half; a = v[m]; b = v[m + half]; }
    const float c = cs[m], s = sn[m];
    return first ? a * c - b * s : b * c + a * s;
}

__device__ __forceinline__ int bias_first_key(int p, int window) { return window > 0 ? max(0, p - window + 1) : 0; }

__device__ __forceinline__ float bias_cap(float s, float cap, float inv_cap) { return cap > 0.f ? cap * tanhf(s * inv_cap) : s; }

// ---------------------------------------------------------------------------------
// prep: grid (T, ceil(items / 4)), 4 warps, a warp per (token, item); items = H query heads, G key heads and, unless the
// values are the keys, G value heads.  qkv [T, ld] float, the projections: the first H * dim + G * dim (+ G * vdim) columns.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void bias_prep_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, const float* __restrict__ qw,
                                 const float* __restrict__ kw, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                 int table_width, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, int H, int G,
                                 int dim, int vdim, int rdims, int interleaved, float eps, int store_kv, int values_are_keys, int ld) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float bufs[4][QWB_BIAS_MAX_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y * 4 + warp, t = blockIdx.x;
    const int n_items = H + G + (values_are_keys ? 0 : G);
    if (item >= n_items) return;
    float* buf = bufs[warp];
    const bool is_q = item < H, is_k = !is_q && item < H + G;
    const int n = (is_q || is_k) ? dim : vdim;
    const int col = is_q ? item * dim : (is_k ? H * dim + (item - H) * dim : (H + G) * dim + (item - H - G) * vdim);
    const float* src = qkv + (size_t)t * ld + col;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) { const float v = src[i] + (bias ? bias[col + i] : 0.f); buf[i] = v; ss += v * v; }
    size_t cache_row = 0;
    if (!is_q) {
        if (!store_kv) return;
        const int b = tok_seq[t], p = tok_pos[t];
        const size_t page = page_table[(size_t)b * table_width + p / QWB_BIAS_PAGE];
        const int head = is_k ? item - H : item - H - G;
        cache_row = (page * G + head) * QWB_BIAS_PAGE + p % QWB_BIAS_PAGE;
        if (!is_k || values_are_keys) {                     // a value row: the projection as it is
            T* vdst = v_pool + cache_row * (size_t)vdim;
            for (int i = lane; i < n; i += 32) vdst[i] = from_f32<T>(buf[i]);
            if (!is_k) return;
        }
    }
    const float* w = is_q ? qw : kw;
    if (w) {
        const float scale = rsqrtf(warp_sum(ss) / (float)n + eps);
        for (int i = lane; i < n; i += 32) buf[i] = buf[i] * scale * w[i];
    }
    __syncwarp();
    const float* cs = cos_t + (size_t)t * (rdims >> 1);
    const float* sn = sin_t + (size_t)t * (rdims >> 1);
    T* dst = is_q ? q_out + ((size_t)t * H + item) * dim : k_pool + cache_row * (size_t)dim;
    for (int i = lane; i < n; i += 32) dst[i] = from_f32<T>(rdims > 0 ? bias_turned(buf, i, rdims, cs, sn, interleaved) : buf[i]);
}

// `step`: 1 for the kernels that read value by value, 8 for those that copy 16 bytes at a time
static int check_bias_sizes(const char* what, int H, int G, int dim, int vdim, int table_width, int window, int step) {
    if (H <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", what, H, G);
    if (dim <= 0 || dim % step || dim > QWB_BIAS_MAX_DIM || vdim <= 0 || vdim % step || vdim > QWB_BIAS_MAX_DIM)
        return qwb_fail(QWB_ERR_ARG, "%s: key size %d or value size %d is not a multiple of %d in [%d, %d]", what, dim, vdim, step, step, QWB_BIAS_MAX_DIM);
    if (table_width <= 0 || window < 0) return qwb_fail(QWB_ERR_ARG, "%s: bad table width %d or window %d", what, table_width, window);
    return 0;
}

extern "C" int qwb_bias_prep(const float* qkv, const float* bias, const float* qw, const float* kw, const float* cos_t, const float* sin_t,
                             const int* tok_seq, const int* tok_pos, const int* page_table, int table_width, void* q_out, void* k_pool,
                             void* v_pool, int dtype, int T, int H, int G, int dim, int vdim, int rdims, int interleaved, float eps,
                             int store_kv, int values_are_keys, int ld, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (int rc = check_bias_sizes("bias_prep", H, G, dim, vdim, table_width, 0, 1)) return rc;
    if (ld < (H + G) * dim + (values_are_keys ? 0 : G * vdim)) return qwb_fail(QWB_ERR_ARG, "bias_prep: rows of %d values do not hold the projections", ld);
    if (values_are_keys && vdim != dim) return qwb_fail(QWB_ERR_ARG, "bias_prep: values that are the keys have their size, not %d for %d", vdim, dim);
    if (rdims < 0 || rdims > dim || rdims % 2) return qwb_fail(QWB_ERR_ARG, "bias_prep: a rotation of %d of %d values", rdims, dim);
    if (rdims > 0 && (!cos_t || !sin_t)) return qwb_fail(QWB_ERR_ARG, "bias_prep: a rotation without its table");
    dim3 grid(T, (H + G + (values_are_keys ? 0 : G) + 3) / 4);
    if (dtype == QWB_DT_F32)
        qwb_launch(bias_prep_kernel<float>, grid, 128, 0, stream, qkv, bias, qw, kw, cos_t, sin_t, tok_seq, tok_pos, page_table, table_width,
                   (float*)q_out, (float*)k_pool, (float*)v_pool, H, G, dim, vdim, rdims, interleaved, eps, store_kv, values_are_keys, ld);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(bias_prep_kernel<bf16>, grid, 128, 0, stream, qkv, bias, qw, kw, cos_t, sin_t, tok_seq, tok_pos, page_table, table_width,
                   (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, H, G, dim, vdim, rdims, interleaved, eps, store_kv, values_are_keys, ld);
    else return qwb_fail(QWB_ERR_ARG, "bias_prep: unknown dtype %d", dtype);
    return qwb_check_launch("bias_prep");
}

// ---------------------------------------------------------------------------------
// prefill: one block per (tile of 16 queries, query head and value head, sequence); 4 warps, each owns 4 queries; keys
// come in tiles of 32 (one key per lane), from the first key that the tile's first query sees to the tile's last query.
// C = G (all_values) or 1 value heads per query head; out [T, H, C, vdim].
// ---------------------------------------------------------------------------------
template <typename T, typename TO, int NC>   // NC = ceil(vdim / 32) rounded up to 2, 4 or 8
__global__ void bias_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                    const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                                    TO* __restrict__ out, int H, int G, int C, int dim, int vdim, int table_width, float scale,
                                    const float* __restrict__ head_scale, float softcap, const float* __restrict__ slopes, int window,
                                    const float* __restrict__ sinks) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BQ = 16, BK = 32, QPW = 4, PG = QWB_BIAS_PAGE;
    extern __shared__ float smem[];
    float* Qs = smem;                         // [BQ][dim], already scaled
    float* Ks = Qs + BQ * dim;                // [BK][dim + 1]
    float* Vs = Ks + BK * (dim + 1);          // [BK][vdim]

    const int b = blockIdx.z, h = blockIdx.y / C, c = blockIdx.y % C, q0 = blockIdx.x * BQ;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    if (q0 >= n_new) return;
    const int g = h / (H / G), vg = C > 1 ? c : g;
    const int p0 = pos0[b];
    const int nq = min(BQ, n_new - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
    const float hs = scale * (head_scale ? head_scale[h] : 1.f);
    const float slope = slopes ? slopes[h] : 0.f;

    const int k_last = p0 + q0 + nq - 1;
    const int k_first = bias_first_key(p0 + q0, window);
    const int* pages = page_table + (size_t)b * table_width;

    for (int idx = threadIdx.x; idx < BQ * dim; idx += blockDim.x) {
        const int i = idx / dim, d = idx - i * dim;
        Qs[idx] = i < nq ? to_f32(q[((size_t)(t0 + q0 + i) * H + h) * dim + d]) * hs : 0.f;
    }
    float m[QPW], l[QPW], acc[QPW][NC];
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) acc[i][cc] = 0.f;
    }
    for (int kt = (k_first / BK) * BK; kt <= k_last; kt += BK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < BK * dim; idx += blockDim.x) {
            const int j = idx / dim, d = idx - j * dim, key = kt + j;
            Ks[j * (dim + 1) + d] = key <= k_last ? to_f32(k_pool[(((size_t)pages[key / PG] * G + g) * PG + key % PG) * dim + d]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BK * vdim; idx += blockDim.x) {
            const int j = idx / vdim, d = idx - j * vdim, key = kt + j;
            Vs[idx] = key <= k_last ? to_f32(v_pool[(((size_t)pages[key / PG] * G + vg) * PG + key % PG) * vdim + d]) : 0.f;
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
            const bool ok = qi < nq && key <= qp && key >= bias_first_key(qp, window);
            const float si = ok ? bias_cap(s[i], softcap, inv_cap) - slope * (float)(qp - key) : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(si));
            if (m_new == -INFINITY) { p[i] = 0.f; continue; }       // nothing visible so far (whole warp agrees)
            const float alpha = expf(m[i] - m_new);                 // m = -inf gives 0
            p[i] = ok ? expf(si - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(p[i]);
            m[i] = m_new;
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) acc[i][cc] *= alpha;
        }
        for (int j = 0; j < BK; ++j) {
            float pj[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) {
                const int d = lane + 32 * cc;
                if (d < vdim) {
                    const float v = Vs[j * vdim + d];
#pragma unroll
                    for (int i = 0; i < QPW; ++i) acc[i][cc] += pj[i] * v;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        if (qi >= nq) continue;
        float li = l[i], mul = 1.f;
        if (sinks) {                                                // one more term of the denominator
            const float sk = sinks[h], m2 = fmaxf(m[i], sk);
            mul = expf(m[i] - m2);
            li = li * mul + expf(sk - m2);
        }
        const float inv = li > 0.f ? mul / li : 0.f;
        TO* o = out + (((size_t)(t0 + q0 + qi) * H + h) * C + c) * vdim;
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
            const int d = lane + 32 * cc;
            if (d < vdim) o[d] = from_f32<TO>(acc[i][cc] * inv);
        }
    }
}

template <typename T, typename TO>
static int launch_bias_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                               const int* pos0, void* out, int B, int max_new, int H, int G, int C, int dim, int vdim, int table_width,
                               float scale, const float* head_scale, float softcap, const float* slopes, int window, const float* sinks,
                               cudaStream_t stream) {
    const size_t smem = ((size_t)16 * dim + 32 * (dim + 1) + 32 * vdim) * sizeof(float);
    dim3 grid((max_new + 15) / 16, H * C, B);
    const int nc = (vdim + 31) / 32;
#define QWB_LAUNCH_BIAS_PREFILL(NC)                                                                              \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(bias_prefill_kernel<T, TO, NC>,                                 \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "bias_prefill: %s", cudaGetErrorString(e));      \
        }                                                                                                        \
        qwb_launch(bias_prefill_kernel<T, TO, NC>, grid, 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, \
            page_table, cu_seqlens, pos0, (TO*)out, H, G, C, dim, vdim, table_width, scale, head_scale, softcap, slopes, window, sinks); \
    } while (0)
    if (nc <= 2) QWB_LAUNCH_BIAS_PREFILL(2);
    else if (nc <= 4) QWB_LAUNCH_BIAS_PREFILL(4);
    else QWB_LAUNCH_BIAS_PREFILL(8);
#undef QWB_LAUNCH_BIAS_PREFILL
    return qwb_check_launch("bias_prefill");
}

// q [T, H, dim]; out [T, H, C, vdim] with C = G (all_values; float) or 1 (raw_out: float, else the cache's dtype).
extern "C" int qwb_bias_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                                const int* pos0, void* out, int dtype, int raw_out, int B, int max_new, int H, int G, int all_values,
                                int dim, int vdim, int table_width, float scale, const float* head_scale, float softcap,
                                const float* slopes, int window, const float* sinks, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_bias_sizes("bias_prefill", H, G, dim, vdim, table_width, window, 1)) return rc;
    const int C = all_values ? G : 1;
    if (all_values && !raw_out) return qwb_fail(QWB_ERR_ARG, "bias_prefill: the outputs for all value heads are 32-bit");
    if (B > 65535 || H * C > 65535) return qwb_fail(QWB_ERR_ARG, "bias_prefill: batch %d or heads %d above 65535", B, H * C);
#define QWB_BIAS_PF(T, TO) launch_bias_prefill<T, TO>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, H, G, C, dim, vdim, \
                                                     table_width, scale, head_scale, softcap, slopes, window, sinks, stream)
    if (dtype == QWB_DT_F32) return QWB_BIAS_PF(float, float);
    if (dtype == QWB_DT_BF16) return raw_out ? QWB_BIAS_PF(bf16, float) : QWB_BIAS_PF(bf16, bf16);
#undef QWB_BIAS_PF
    return qwb_fail(QWB_ERR_ARG, "bias_prefill: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// prefill on the tensor cores (bfloat16, mma.sync m16n8k16): block = 64 queries of one (sequence, query head, value
// head), 4 warps of 16 rows; keys in tiles of 64 = one page of the cache, from the page of the first key that the tile's
// first query sees to the page of its last query.  Q, K and V tiles sit in shared memory with rows padded by 16 bytes
// (conflict-free ldmatrix); K has two buffers, V one: the next tile's keys are copied in (cp.async) under this tile's work,
// its values under its own scores and softmax.  Scores, the cap, the distance bias, maxima, sums, the sink and the
// accumulators are 32-bit; probabilities are rounded to bfloat16 for the second product.  dim a multiple of 16, vdim of 8.
// ---------------------------------------------------------------------------------
#define BM_BQ 64
#define BM_BK 64
#define BM_PAD 8

__device__ __forceinline__ void bm_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void bm_ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void bm_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; `bytes` 0 writes zeros (src must still be a valid address)
__device__ __forceinline__ void bm_cp16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void bm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t bm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float bm_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void bm_store2(bf16* p, float a, float b) { *reinterpret_cast<uint32_t*>(p) = bm_pack(a, b); }
__device__ __forceinline__ void bm_store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
// 16-byte pieces of a [rows][cpr pieces] tile, dealt to 128 threads in order: the thread's first piece and its stride,
// as (row, piece) pairs, so that the copy loops divide nothing
struct BmWalk {
    int r0, c0, dr, dc, cpr;
    __device__ __forceinline__ BmWalk(int tid, int pieces_per_row) : r0(tid / pieces_per_row), c0(tid % pieces_per_row),
        dr(128 / pieces_per_row), dc(128 % pieces_per_row), cpr(pieces_per_row) {}
    __device__ __forceinline__ void next(int& r, int& c) const { r += dr; c += dc; if (c >= cpr) { c -= cpr; ++r; } }
};

template <int NV, typename TO>     // n-tiles of 8 value columns the accumulator has room for; the output's type
__global__ void __launch_bounds__(128)
bias_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                        TO* __restrict__ out, int H, int G, int C, int dim, int vdim, int table_width, float scale,
                        const float* __restrict__ head_scale, float softcap, const float* __restrict__ slopes, int window,
                        const float* __restrict__ sinks) {
    pdl_wait();
    pdl_launch_dependents();
    const int ldq = dim + BM_PAD, ldv = vdim + BM_PAD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Kbuf = Qs + BM_BQ * ldq;                          // [2][64][ldq]
    bf16* Vbuf = Kbuf + 2 * BM_BK * ldq;                    // [64][ldv]

    // the last queries see the most keys: their blocks start first, so that the long blocks are not the launch's tail
    const int b = blockIdx.z, h = blockIdx.y / C, c = blockIdx.y % C, q0 = (int)(gridDim.x - 1 - blockIdx.x) * BM_BQ;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (q0 >= n) return;
    const int g_kv = h / (H / G), g_v = C > 1 ? c : g_kv;
    const int p0 = pos0[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = min(BM_BQ, n - q0);
    const int gr = lane >> 2, tq = lane & 3;
    const int pos_a = p0 + q0 + warp * 16 + gr, pos_b = pos_a + 8;  // positions of the thread's two rows
    const int lo_a = bias_first_key(pos_a, window), lo_b = bias_first_key(pos_b, window);

    const int k_hi = p0 + q0 + nq - 1;                              // last key any query of the tile sees
    const int k_lo = bias_first_key(p0 + q0, window);               // first key any of them sees
    const int nv_used = vdim / 8;
    const int first_page = k_lo / BM_BK, n_tiles = k_hi / BM_BK - first_page + 1;
    const int* pages = page_table + (size_t)b * table_width;
    const int warp_lo = p0 + q0 + warp * 16, warp_hi = warp_lo + 15;
    const int warp_first = bias_first_key(warp_hi, window);         // the first key that every row of the warp may see
    const float log2e = 1.4426950408889634f;
    // Scores in units of ln 2 (ex2 below).  With a cap c: c tanh(x / c) = c - 2 c / (e^(2 x / c) + 1), exact at both ends
    // (e^.. = inf or 0) and a few units of the last place in between: one ex2, one rcp and one fma a score.
    const float hs = scale * (head_scale ? head_scale[h] : 1.f);
    const float mul_s = softcap > 0.f ? hs / softcap * 2.f * log2e : hs * log2e;
    const float cap2 = softcap * log2e;
    const float slope2 = slopes ? slopes[h] * log2e : 0.f;
    const BmWalk walk_k(tid, dim / 8), walk_v(tid, vdim / 8);

    auto copy_keys = [&](int it, int stage) {                   // one commit group
        const int page = first_page + it;
        const int rows = min(BM_BK, k_hi + 1 - page * BM_BK);
        const bf16* ks = k_pool + ((size_t)pages[page] * G + g_kv) * BM_BK * dim;
        bf16* Kd = Kbuf + stage * BM_BK * ldq;
        for (int r = walk_k.r0, cc = walk_k.c0; r < BM_BK; walk_k.next(r, cc))
            bm_cp16(Kd + r * ldq + cc * 8, ks + (size_t)(r < rows ? r : 0) * dim + cc * 8, r < rows ? 16 : 0);
        bm_commit();
    };
    auto copy_values = [&](int it) {                            // one commit group
        const int page = first_page + it;
        const int rows = min(BM_BK, k_hi + 1 - page * BM_BK);
        const bf16* vs = v_pool + ((size_t)pages[page] * G + g_v) * BM_BK * vdim;
        for (int r = walk_v.r0, cc = walk_v.c0; r < BM_BK; walk_v.next(r, cc))
            bm_cp16(Vbuf + r * ldv + cc * 8, vs + (size_t)(r < rows ? r : 0) * vdim + cc * 8, r < rows ? 16 : 0);
        bm_commit();
    };
    for (int r = walk_k.r0, cc = walk_k.c0; r < BM_BQ; walk_k.next(r, cc)) {
        const bool in = r < nq;
        bm_cp16(Qs + r * ldq + cc * 8, q + ((size_t)(t0 + (in ? q0 + r : 0)) * H + h) * dim + cc * 8, in ? 16 : 0);
    }
    // groups in the order of their commits: [Q, K0], V0, K1, V1, K2, ...
    copy_keys(0, 0);
    copy_values(0);

    float o[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows gr and gr + 8 of the warp's 16

    for (int it = 0; it < n_tiles; ++it) {
        const bf16* Ks = Kbuf + (it & 1) * BM_BK * ldq;
        const bf16* Vs = Vbuf;
        const bool more = it + 1 < n_tiles;
        if (more) {                                             // the next keys into the other buffer (its last readers
            copy_keys(it + 1, (it + 1) & 1);                    // passed the barrier at the end of the round before)
            bm_wait<2>();                                       // this tile's keys (and Q) are there
        } else {
            bm_wait<1>();
        }
        __syncthreads();
        const int key0 = (first_page + it) * BM_BK;
        // a tile that no row of the warp sees (behind its last row, or before its window) is skipped by the warp
        const bool none = key0 > warp_hi || key0 + BM_BK <= bias_first_key(warp_lo, window);
        float s[8][4];
        if (!none) {
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            for (int d = 0; d < dim; d += 16) {
                uint32_t a0, a1, a2, a3;
                bm_ldsm_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + d + (lane >> 4) * 8);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {                // two tiles of 8 keys a load
                    uint32_t b0, b1, b2, b3;
                    bm_ldsm_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane & 7) + (lane >> 4) * 8) * ldq + d + ((lane >> 3) & 1) * 8);
                    bm_mma(s[j], a0, a1, a2, a3, b0, b1);
                    bm_mma(s[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            // a tile that every row of the warp sees whole needs no mask (most tiles of a long prompt)
            const bool whole = key0 + BM_BK - 1 <= warp_lo && key0 >= warp_first;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + tq * 2 + (e & 1);
                    bool ok = true;
                    if (!whole) ok = key <= (e < 2 ? pos_a : pos_b) && key >= (e < 2 ? lo_a : lo_b) && key <= k_hi;
                    float v = s[j][e] * mul_s;
                    if (softcap > 0.f) v = fmaf(-2.f * cap2, bm_rcp(bm_ex2(v) + 1.f), cap2);
                    v = fmaf(-slope2, (float)((e < 2 ? pos_a : pos_b) - key), v);
                    s[j][e] = ok ? v : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
            const float alpha0 = bm_ex2(m0 - base0), alpha1 = bm_ex2(m1 - base1);  // m = -inf gives 0
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][0] = bm_ex2(s[j][0] - base0); s[j][1] = bm_ex2(s[j][1] - base0);
                s[j][2] = bm_ex2(s[j][2] - base1); s[j][3] = bm_ex2(s[j][3] - base1);
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

        if (more) bm_wait<1>(); else bm_wait<0>();              // this tile's values are there
        __syncthreads();
        if (!none) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {                    // O += P V, 16 keys a step
                const uint32_t a0 = bm_pack(s[2 * ks][0], s[2 * ks][1]), a1 = bm_pack(s[2 * ks][2], s[2 * ks][3]);
                const uint32_t a2 = bm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = bm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                for (int j = 0; j < NV; j += 2) {
                    if (j < nv_used) {                          // vdim / 8 may be odd: the second tile of a pair reads padding
                        uint32_t b0, b1, b2, b3;                // or the next row's start, and its result is never stored
                        bm_ldsm_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + j * 8 + (lane >> 4) * 8);
                        bm_mma(o[j], a0, a1, a2, a3, b0, b1);
                        if (j + 1 < NV) bm_mma(o[j + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
        }
        __syncthreads();                                        // the values' buffer may be copied into again
        if (more) copy_values(it + 1);
    }

    float mul0 = 1.f, mul1 = 1.f;
    if (sinks) {                                                // one more term of the denominator
        const float sk = sinks[h] * log2e;
        const float n0 = fmaxf(m0, sk), n1 = fmaxf(m1, sk);
        mul0 = bm_ex2(m0 - n0); mul1 = bm_ex2(m1 - n1);
        l0 = l0 * mul0 + bm_ex2(sk - n0); l1 = l1 * mul1 + bm_ex2(sk - n1);
    }
    const float inv0 = l0 > 0.f ? mul0 / l0 : 0.f, inv1 = l1 > 0.f ? mul1 / l1 : 0.f;
    const int row_a = warp * 16 + gr, row_b = row_a + 8;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        if (j < nv_used) {
            const int col = j * 8 + tq * 2;
            if (row_a < nq) bm_store2(out + (((size_t)(t0 + q0 + row_a) * H + h) * C + c) * vdim + col, o[j][0] * inv0, o[j][1] * inv0);
            if (row_b < nq) bm_store2(out + (((size_t)(t0 + q0 + row_b) * H + h) * C + c) * vdim + col, o[j][2] * inv1, o[j][3] * inv1);
        }
    }
}

// Q and two key buffers [64][dim + 8] and one value buffer [64][vdim + 8] of bfloat16
static size_t bm_smem_bytes(int dim, int vdim) {
    return ((size_t)3 * BM_BK * (dim + BM_PAD) + (size_t)BM_BK * (vdim + BM_PAD)) * sizeof(bf16);
}

extern "C" int qwb_bias_prefill_mma_fits(int dtype, int dim, int vdim) {
    return dtype == QWB_DT_BF16 && dim > 0 && dim % 16 == 0 && vdim > 0 && vdim % 8 == 0 && dim <= QWB_BIAS_MAX_DIM &&
           vdim <= QWB_BIAS_MAX_DIM && bm_smem_bytes(dim, vdim) <= 220 * 1024;
}

// q [T, H, dim] bfloat16; out [T, H, C, vdim] as for the plain kernel.
extern "C" int qwb_bias_prefill_mma(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                                    const int* pos0, void* out, int raw_out, int B, int max_new, int H, int G, int all_values, int dim,
                                    int vdim, int table_width, float scale, const float* head_scale, float softcap, const float* slopes,
                                    int window, const float* sinks, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_bias_sizes("bias_prefill_mma", H, G, dim, vdim, table_width, window, 8)) return rc;
    if (!qwb_bias_prefill_mma_fits(QWB_DT_BF16, dim, vdim))
        return qwb_fail(QWB_ERR_ARG, "bias_prefill_mma: keys of %d (a multiple of 16) and values of %d (of 8) that fit in shared memory", dim, vdim);
    const int C = all_values ? G : 1;
    if (all_values && !raw_out) return qwb_fail(QWB_ERR_ARG, "bias_prefill_mma: the outputs for all value heads are 32-bit");
    if (B > 65535 || H * C > 65535) return qwb_fail(QWB_ERR_ARG, "bias_prefill_mma: batch %d or heads %d above 65535", B, H * C);
    for (const void* p : {q, k_pool, v_pool, (const void*)out})
        if ((uintptr_t)p % 16) return qwb_fail(QWB_ERR_ARG, "bias_prefill_mma: a tensor is not 16-byte aligned");
    const size_t smem = bm_smem_bytes(dim, vdim);
    const dim3 grid((max_new + BM_BQ - 1) / BM_BQ, H * C, B);
#define QWB_BM(NV, TO)                                                                                                          \
    do {                                                                                                                        \
        if (smem > 48 * 1024) {                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(bias_prefill_mma_kernel<NV, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "bias_prefill_mma: %s", cudaGetErrorString(e));                 \
        }                                                                                                                       \
        qwb_launch(bias_prefill_mma_kernel<NV, TO>, grid, 128, smem, stream, (const bf16*)q, (const bf16*)k_pool,               \
                   (const bf16*)v_pool, page_table, cu_seqlens, pos0, (TO*)out, H, G, C, dim, vdim, table_width, scale, head_scale, \
                   softcap, slopes, window, sinks);                                                                             \
    } while (0)
#define QWB_BM_SIZES(TO)                                                                                                        \
    do {                                                                                                                        \
        if (vdim <= 32) QWB_BM(4, TO); else if (vdim <= 64) QWB_BM(8, TO); else if (vdim <= 128) QWB_BM(16, TO);                \
        else QWB_BM(32, TO);                                                                                                    \
    } while (0)
    if (raw_out) QWB_BM_SIZES(float); else QWB_BM_SIZES(bf16);
#undef QWB_BM_SIZES
#undef QWB_BM
    return qwb_check_launch("bias_prefill_mma");
}

// ---------------------------------------------------------------------------------
// decode: one new token per sequence (its position is len - 1).  The keys it sees, first .. len - 1 with first the start
// of its window (or 0), are cut into runs of whole pages counted from the page of the first key: 2 pages a run, doubled
// while that would give more than 64 runs.  Which keys a run holds follows from the sequence's own length alone.
// Block = (run, key head, slice of its query heads and value head, sequence), 128 threads; up to 8 query heads a block:
// a page's K and V tiles go to shared memory; thread (key, half of the rows) forms the scores; a warp per row updates
// maximum and sum; thread d accumulates p v for all rows.
// ---------------------------------------------------------------------------------
__device__ __host__ __forceinline__ int bias_run_pages(int first_key, int len) {
    const int span = (len - 1) / QWB_BIAS_PAGE - first_key / QWB_BIAS_PAGE + 1;
    int rp = QWB_BIAS_RUN_PAGES;
    while (span > rp * QWB_BIAS_MAX_RUNS) rp *= 2;
    return rp;
}

__device__ __forceinline__ void bias_cp16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}

template <typename T>
__global__ void bias_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                   const int* __restrict__ page_table, const int* __restrict__ seq_len, float* __restrict__ part_acc,
                                   float* __restrict__ part_m, float* __restrict__ part_l, int H, int G, int C, int dim, int vdim,
                                   int table_width, float scale, const float* __restrict__ head_scale, float softcap,
                                   const float* __restrict__ slopes, int window, int n_runs, int stats_only) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int RT = QWB_BIAS_ROWS, VEC = Vec16<T>::N, PG = QWB_BIAS_PAGE;
    const int b = blockIdx.z, run = blockIdx.x;
    const int len = seq_len[b];
    const int first = bias_first_key(len - 1, window);
    const int rp = bias_run_pages(first, len);
    const int page_lo = first / PG;
    const int row_first = max(first, (page_lo + run * rp) * PG);
    const int row_end = min(len, (page_lo + (run + 1) * rp) * PG);
    if (row_first >= row_end) return;

    const int QG = H / G, slices = (QG + RT - 1) / RT;
    const int c = blockIdx.y % C, gs = blockIdx.y / C;
    const int g = gs / slices, r0 = (gs % slices) * RT;       // query heads g * QG + r0 ... of this key head
    const int rcount = min(RT, QG - r0);
    const int vg = C > 1 ? c : g;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kld = dim + VEC;                          // a key row and 16 bytes: rows start in different banks
    T* Kt = reinterpret_cast<T*>(smem_raw);             // [PG][dim + VEC]
    T* Vt = Kt + (size_t)PG * kld;                      // [PG][vdim]
    float* qs = reinterpret_cast<float*>(Vt + (size_t)PG * vdim);   // [RT][dim], scaled
    float* sc = qs + RT * dim;                          // [RT][PG]
    float* m_s = sc + RT * PG;                          // [RT]
    float* l_s = m_s + RT;
    float* a_s = l_s + RT;
    float* sl_s = a_s + RT;                             // the rows' slopes

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head0 = g * QG + r0;
    const T* qrow = q + ((size_t)b * H + head0) * dim;
    for (int idx = tid; idx < RT * dim; idx += blockDim.x) {
        const int ri = idx / dim;
        qs[idx] = ri < rcount ? to_f32(qrow[idx]) * scale * (head_scale ? head_scale[head0 + ri] : 1.f) : 0.f;
    }
    if (tid < RT) {
        m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f;
        sl_s[tid] = (slopes && tid < rcount) ? slopes[head0 + tid] : 0.f;
    }

    float acc[RT][2];
#pragma unroll
    for (int ri = 0; ri < RT; ++ri) acc[ri][0] = acc[ri][1] = 0.f;

    const int* pages = page_table + (size_t)b * table_width;
    const int my_key = tid % PG, my_slice = tid / PG;                 // two threads a key; each takes every second row
    const int dchunk = dim / VEC;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

    for (int base = (row_first / PG) * PG; base < row_end; base += PG) {
        const int n_keys = min(PG, row_end - base);
        __syncthreads();                                              // the last page's tiles are no longer read
        {
            const size_t page = (size_t)pages[base / PG];
            const uint4* ksrc = reinterpret_cast<const uint4*>(k_pool + (page * G + g) * PG * dim);
            const uint4* vsrc = reinterpret_cast<const uint4*>(v_pool + (page * G + vg) * PG * vdim);
            uint4* kdst = reinterpret_cast<uint4*>(Kt);
            uint4* vdst = reinterpret_cast<uint4*>(Vt);
            for (int i = tid; i < n_keys * dchunk; i += blockDim.x) bias_cp16(kdst + i + i / dchunk, ksrc + i);     // row r starts at r * (dchunk + 1)
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (!stats_only)
                for (int i = tid; i < n_keys * vdim / VEC; i += blockDim.x) bias_cp16(vdst + i, vsrc + i);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");     // the keys are there; the values arrive under the scores
        }
        __syncthreads();

        if (my_key < n_keys) {
            const Vec16<T>* krow = reinterpret_cast<const Vec16<T>*>(Kt + (size_t)my_key * kld);
            const bool ok = base + my_key >= row_first;
            const float dist = (float)(len - 1 - (base + my_key));
            float s[RT / 2];
#pragma unroll
            for (int k = 0; k < RT / 2; ++k) s[k] = 0.f;
            for (int ch = 0; ch < dchunk; ++ch) {
                float kf[VEC];
                krow[ch].get(kf);
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
                if (ri < rcount) sc[ri * PG + my_key] = ok ? bias_cap(s[k], softcap, inv_cap) - sl_s[ri] * dist : -INFINITY;
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
        if (stats_only) continue;                                     // maxima and sums only: the values are not read

#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const int d = tid + cc * 128;
            if (d < vdim) {
#pragma unroll
                for (int ri = 0; ri < RT; ++ri) if (ri < rcount) acc[ri][cc] *= a_s[ri];
                int j = 0;
                for (; j + 4 <= n_keys; j += 4) {                    // four keys' weights of a row in one load
                    const float v0 = to_f32(Vt[(size_t)j * vdim + d]), v1 = to_f32(Vt[(size_t)(j + 1) * vdim + d]);
                    const float v2 = to_f32(Vt[(size_t)(j + 2) * vdim + d]), v3 = to_f32(Vt[(size_t)(j + 3) * vdim + d]);
#pragma unroll
                    for (int ri = 0; ri < RT; ++ri)
                        if (ri < rcount) {
                            const float4 p = *reinterpret_cast<const float4*>(sc + ri * PG + j);
                            acc[ri][cc] += p.x * v0 + p.y * v1 + p.z * v2 + p.w * v3;
                        }
                }
                for (; j < n_keys; ++j) {
                    const float v = to_f32(Vt[(size_t)j * vdim + d]);
#pragma unroll
                    for (int ri = 0; ri < RT; ++ri) if (ri < rcount) acc[ri][cc] += sc[ri * PG + j] * v;
                }
            }
        }
    }
    __syncthreads();

#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int d = tid + cc * 128;
        if (d >= vdim || stats_only) continue;
#pragma unroll
        for (int ri = 0; ri < RT; ++ri)
            if (ri < rcount) part_acc[((((size_t)b * H + head0 + ri) * C + c) * n_runs + run) * vdim + d] = acc[ri][cc];
    }
    if (tid < rcount) {
        const size_t at = (((size_t)b * H + head0 + tid) * C + c) * n_runs + run;
        part_m[at] = m_s[tid];
        part_l[at] = l_s[tid];
    }
}

// Per (query head, value head, sequence): a = sum_r acc_r e^(m_r - M) / (sum_r l_r e^(m_r - M) + e^(sink - M)), M the
// largest of the runs' maxima and the sink, over the sequence's runs in index order.  grid (H * C, B), 128 threads: warp 0
// first makes the weights e^(m_r - M) / L once for all columns, then thread d sums its column.
template <typename TO>
__global__ void bias_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m, const float* __restrict__ part_l,
                                  const int* __restrict__ seq_len, TO* __restrict__ out, int C, int vdim, int window, int n_runs,
                                  const float* __restrict__ sinks) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float wts[QWB_BIAS_MAX_RUNS];
    const int hc = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const size_t row = (size_t)b * gridDim.x + hc;
    const int len = seq_len[b];
    const int first = bias_first_key(len - 1, window);
    const int rp = bias_run_pages(first, len);
    const int runs = min(n_runs, ((len - 1) / QWB_BIAS_PAGE - first / QWB_BIAS_PAGE) / rp + 1);
    if (tid < 32) {
        float M = sinks ? sinks[hc / C] : -INFINITY;
        for (int r = lane; r < runs; r += 32) M = fmaxf(M, part_m[row * n_runs + r]);
        M = warp_max(M);
        float L = 0.f;
        for (int r = lane; r < runs; r += 32) {
            const float e = M == -INFINITY ? 0.f : expf(part_m[row * n_runs + r] - M);
            wts[r] = e;
            L += part_l[row * n_runs + r] * e;
        }
        L = warp_sum(L);
        if (sinks) L += expf(sinks[hc / C] - M);
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int r = lane; r < runs; r += 32) wts[r] *= inv;
    }
    __syncthreads();
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int d = tid + cc * 128;
        if (d >= vdim) continue;
        const float* col = part_acc + row * n_runs * vdim + d;
        float a = 0.f;
#pragma unroll 8
        for (int r = 0; r < runs; ++r) a += col[(size_t)r * vdim] * wts[r];
        out[row * vdim + d] = from_f32<TO>(a);
    }
}

// runs of the grid for sequences of up to max_len tokens
extern "C" int qwb_bias_decode_runs(int max_len, int window) {
    if (max_len <= 0) return 1;
    // the most pages a sequence's visible keys touch: a window may begin anywhere in its first page
    const int pages_all = (max_len + QWB_BIAS_PAGE - 1) / QWB_BIAS_PAGE;
    const int pages = window > 0 ? min(pages_all, (window + QWB_BIAS_PAGE - 2) / QWB_BIAS_PAGE + 1) : pages_all;
    const int runs = (pages + QWB_BIAS_RUN_PAGES - 1) / QWB_BIAS_RUN_PAGES;
    return runs < QWB_BIAS_MAX_RUNS ? runs : QWB_BIAS_MAX_RUNS;
}

extern "C" long long qwb_bias_decode_scratch_floats(int B, int H, int C, int vdim, int n_runs) {
    return (long long)B * H * C * n_runs * (vdim + 2);
}

template <typename T, typename TO>
static int launch_bias_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                              float* scratch, void* out, int B, int H, int G, int C, int dim, int vdim, int table_width, float scale,
                              const float* head_scale, float softcap, const float* slopes, int window, const float* sinks, int n_runs,
                              cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    const size_t rows = (size_t)B * H * C;
    float* part_acc = scratch;
    float* part_m = part_acc + rows * n_runs * vdim;
    float* part_l = part_m + rows * n_runs;
    const size_t smem = ((size_t)QWB_BIAS_PAGE * (dim + VEC) + (size_t)QWB_BIAS_PAGE * vdim) * sizeof(T) +
                        ((size_t)QWB_BIAS_ROWS * dim + QWB_BIAS_ROWS * QWB_BIAS_PAGE + 4 * QWB_BIAS_ROWS) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(bias_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "bias_decode: %s", cudaGetErrorString(e));
    }
    const int slices = (H / G + QWB_BIAS_ROWS - 1) / QWB_BIAS_ROWS;
    qwb_launch(bias_decode_kernel<T>, dim3(n_runs, G * slices * C, B), 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool,
               page_table, seq_len, part_acc, part_m, part_l, H, G, C, dim, vdim, table_width, scale, head_scale, softcap, slopes, window,
               n_runs, 0);
    if (int rc = qwb_check_launch("bias_decode")) return rc;
    qwb_launch(bias_merge_kernel<TO>, dim3(H * C, B), 128, 0, stream, (const float*)part_acc, (const float*)part_m, (const float*)part_l,
               seq_len, (TO*)out, C, vdim, window, n_runs, sinks);
    return qwb_check_launch("bias_merge");
}

// q [B, H, dim]; out [B, H, C, vdim] as for the prefill kernel; scratch: qwb_bias_decode_scratch_floats floats.
extern "C" int qwb_bias_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                               float* scratch, void* out, int dtype, int raw_out, int B, int H, int G, int all_values, int dim, int vdim,
                               int table_width, float scale, const float* head_scale, float softcap, const float* slopes, int window,
                               const float* sinks, int n_runs, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (int rc = check_bias_sizes("bias_decode", H, G, dim, vdim, table_width, window, 8)) return rc;
    const int C = all_values ? G : 1;
    if (all_values && !raw_out) return qwb_fail(QWB_ERR_ARG, "bias_decode: the outputs for all value heads are 32-bit");
    if (n_runs <= 0 || n_runs > 65535 || B > 65535) return qwb_fail(QWB_ERR_ARG, "bias_decode: %d runs, %d sequences", n_runs, B);
#define QWB_BIAS_DEC(T, TO) launch_bias_decode<T, TO>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, H, G, C, dim, vdim, table_width, \
                                                     scale, head_scale, softcap, slopes, window, sinks, n_runs, stream)
    if (dtype == QWB_DT_F32) return QWB_BIAS_DEC(float, float);
    if (dtype == QWB_DT_BF16) return raw_out ? QWB_BIAS_DEC(bf16, float) : QWB_BIAS_DEC(bf16, bf16);
#undef QWB_BIAS_DEC
    return qwb_fail(QWB_ERR_ARG, "bias_decode: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// decode with mixed heads in two passes over the keys.  The mix needs every head's NORMALISED weights, so the first
// pass (the decode kernel above without its values) leaves each run's maxima and sums, bias_stats_kernel turns them
// into each head's maximum M and 1 / denominator (with the sink), and the second pass, one block per (run, sequence) for
// ALL heads, forms for a page of keys every head's weights e^(s - M) / L in shared memory, mixes them there,
// w'_h = sum_g mix[h, g] w_g, and adds w'_h times the values of h's own value head onto its sums: keys twice and values
// once, where the form with all value heads reads the keys and forms the scores once per value head.  The runs' sums
// simply add up (the weights are final), which bias_mixed_merge does, with the gate.
// ---------------------------------------------------------------------------------
#define QWB_BIAS_MIXED_THREADS 256
#define QWB_BIAS_MIXED_ACC 16      // sums a thread keeps: H * vdim <= 256 * 16

// grid (H, B), 32 threads: stats [B, H, 2] = the maximum (of the runs and the sink) and 1 / denominator
__global__ void bias_stats_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l, const int* __restrict__ seq_len,
                                  float* __restrict__ stats, int window, int n_runs, const float* __restrict__ sinks) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
    const size_t row = (size_t)b * gridDim.x + h;
    const int len = seq_len[b];
    const int first = bias_first_key(len - 1, window);
    const int rp = bias_run_pages(first, len);
    const int runs = min(n_runs, ((len - 1) / QWB_BIAS_PAGE - first / QWB_BIAS_PAGE) / rp + 1);
    float M = sinks ? sinks[h] : -INFINITY;
    for (int r = lane; r < runs; r += 32) M = fmaxf(M, part_m[row * n_runs + r]);
    M = warp_max(M);
    float L = 0.f;
    for (int r = lane; r < runs; r += 32) L += part_l[row * n_runs + r] * (M == -INFINITY ? 0.f : expf(part_m[row * n_runs + r] - M));
    L = warp_sum(L);
    if (sinks) L += expf(sinks[h] - M);
    if (lane == 0) { stats[2 * row] = M; stats[2 * row + 1] = L > 0.f ? 1.f / L : 0.f; }
}

__device__ __forceinline__ void bias_load2(const float* p, float& a, float& b) { const float2 v = *reinterpret_cast<const float2*>(p); a = v.x; b = v.y; }
__device__ __forceinline__ void bias_load2(const bf16* p, float& a, float& b) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
}

template <typename T>
__global__ void __launch_bounds__(QWB_BIAS_MIXED_THREADS)
bias_decode_mixed_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int* __restrict__ page_table, const int* __restrict__ seq_len, const float* __restrict__ stats,
                         const float* __restrict__ mix, float* __restrict__ part, int H, int G, int dim, int vdim, int table_width,
                         float scale, const float* __restrict__ head_scale, float softcap, const float* __restrict__ slopes, int window,
                         int n_runs) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int VEC = Vec16<T>::N, PG = QWB_BIAS_PAGE, NT = QWB_BIAS_MIXED_THREADS, NA = QWB_BIAS_MIXED_ACC, RT = QWB_BIAS_ROWS;
    const int b = blockIdx.y, run = blockIdx.x;
    const int len = seq_len[b];
    const int first = bias_first_key(len - 1, window);
    const int rp = bias_run_pages(first, len);
    const int page_lo = first / PG;
    const int row_first = max(first, (page_lo + run * rp) * PG);
    const int row_end = min(len, (page_lo + (run + 1) * rp) * PG);
    float* out = part + ((size_t)b * n_runs + run) * H * vdim;
    const int tid = threadIdx.x;
    if (row_first >= row_end) {                                      // a run without keys adds nothing
        for (int i = tid; i < H * vdim; i += NT) out[i] = 0.f;
        return;
    }
    const int QG = H / G;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kld = dim + VEC;
    const size_t tile_elems = (size_t)G * PG * (kld > vdim ? kld : vdim);
    T* tile = reinterpret_cast<T*>(smem_raw);                        // the keys of all key heads [G][PG][dim + VEC], then the values [G][PG][vdim]
    float* qs = reinterpret_cast<float*>(tile + tile_elems);         // [H][dim], scaled
    float* w = qs + (size_t)H * dim;                                 // [H][PG] normalised weights
    float* w2 = w + (size_t)H * PG;                                  // [H][PG] mixed
    float* mx = w2 + (size_t)H * PG;                                 // [H][H]
    float* st = mx + (size_t)H * H;                                  // [H][3]: maximum, 1 / denominator, slope

    for (int idx = tid; idx < H * dim; idx += NT) {
        const int h = idx / dim;
        qs[idx] = to_f32(q[(size_t)b * H * dim + idx]) * scale * (head_scale ? head_scale[h] : 1.f);
    }
    for (int idx = tid; idx < H * H; idx += NT) mx[idx] = mix[idx];
    for (int h = tid; h < H; h += NT) {
        st[3 * h] = stats[2 * ((size_t)b * H + h)];
        st[3 * h + 1] = stats[2 * ((size_t)b * H + h) + 1];
        st[3 * h + 2] = slopes ? slopes[h] : 0.f;
    }
    float acc[NA];
#pragma unroll
    for (int i = 0; i < NA; ++i) acc[i] = 0.f;

    const int* pages = page_table + (size_t)b * table_width;
    const int dchunk = dim / VEC;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

    for (int base = (row_first / PG) * PG; base < row_end; base += PG) {
        const int n_keys = min(PG, row_end - base);
        const size_t page = (size_t)pages[base / PG];
        __syncthreads();                                              // the last page's values are no longer read
        for (int i = tid; i < G * n_keys * dchunk; i += NT) {
            const int g = i / (n_keys * dchunk), rest = i - g * n_keys * dchunk, r = rest / dchunk, ch = rest - r * dchunk;
            bias_cp16(tile + ((size_t)g * PG + r) * kld + ch * VEC, k_pool + ((page * G + g) * PG + r) * (size_t)dim + ch * VEC);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // every head's weights for the page's keys: a thread takes a key of a key head and up to 8 of its query heads at a time
        for (int item = tid; item < G * PG; item += NT) {
            const int g = item / PG, key = item - g * PG;
            const bool ok = key < n_keys && base + key >= row_first;
            const float dist = (float)(len - 1 - (base + key));
            const Vec16<T>* krow = reinterpret_cast<const Vec16<T>*>(tile + ((size_t)g * PG + key) * kld);
            for (int h0 = 0; h0 < QG; h0 += RT) {
                float s[RT];
#pragma unroll
                for (int k = 0; k < RT; ++k) s[k] = 0.f;
                if (ok) {
                    for (int ch = 0; ch < dchunk; ++ch) {
                        float kf[VEC];
                        krow[ch].get(kf);
#pragma unroll
                        for (int k = 0; k < RT; ++k) {
                            if (h0 + k < QG) {
                                const float4* qr = reinterpret_cast<const float4*>(qs + (size_t)(g * QG + h0 + k) * dim + ch * VEC);
#pragma unroll
                                for (int e = 0; e < VEC / 4; ++e) {
                                    const float4 qv = qr[e];
                                    s[k] += qv.x * kf[4 * e] + qv.y * kf[4 * e + 1] + qv.z * kf[4 * e + 2] + qv.w * kf[4 * e + 3];
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int k = 0; k < RT; ++k) {
                    if (h0 + k < QG) {
                        const int h = g * QG + h0 + k;
                        w[h * PG + key] = ok ? expf(bias_cap(s[k], softcap, inv_cap) - st[3 * h + 2] * dist - st[3 * h]) * st[3 * h + 1] : 0.f;
                    }
                }
            }
        }
        __syncthreads();                                              // the keys are no longer read: the values may come
        for (int i = tid; i < G * n_keys * (vdim / VEC); i += NT) {
            const int per = n_keys * (vdim / VEC), g = i / per, rest = i - g * per;
            bias_cp16(tile + (size_t)g * PG * vdim + (size_t)rest * VEC, v_pool + (page * G + g) * PG * (size_t)vdim + (size_t)rest * VEC);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        for (int idx = tid; idx < H * PG; idx += NT) {                // the mix, under the values' copy
            const int h = idx / PG, key = idx - h * PG;
            float v = 0.f;
            for (int g2 = 0; g2 < H; ++g2) v += mx[h * H + g2] * w[g2 * PG + key];
            w2[idx] = v;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // a thread keeps pairs of neighbouring value columns: four keys' weights in one load, two values in one
        const int half = vdim >> 1;
#pragma unroll
        for (int i = 0; i < NA / 2; ++i) {
            const int idx = tid + i * NT;
            if (idx < H * half) {
                const int h = idx / half, d = (idx - h * half) * 2;
                const T* vcol = tile + (size_t)(h / QG) * PG * vdim + d;
                const float* wr = w2 + h * PG;
                float a0 = acc[2 * i], a1 = acc[2 * i + 1];
                int j = 0;
                for (; j + 4 <= n_keys; j += 4) {
                    const float4 p = *reinterpret_cast<const float4*>(wr + j);
                    float x0, y0, x1, y1, x2, y2, x3, y3;
                    bias_load2(vcol + (size_t)j * vdim, x0, y0);
                    bias_load2(vcol + (size_t)(j + 1) * vdim, x1, y1);
                    bias_load2(vcol + (size_t)(j + 2) * vdim, x2, y2);
                    bias_load2(vcol + (size_t)(j + 3) * vdim, x3, y3);
                    a0 += p.x * x0 + p.y * x1 + p.z * x2 + p.w * x3;
                    a1 += p.x * y0 + p.y * y1 + p.z * y2 + p.w * y3;
                }
                for (; j < n_keys; ++j) {
                    float x, y;
                    bias_load2(vcol + (size_t)j * vdim, x, y);
                    a0 += wr[j] * x; a1 += wr[j] * y;
                }
                acc[2 * i] = a0; acc[2 * i + 1] = a1;
            }
        }
    }
    const int half = vdim >> 1;
#pragma unroll
    for (int i = 0; i < NA / 2; ++i) {
        const int idx = tid + i * NT;
        if (idx < H * half) {
            const int h = idx / half, d = (idx - h * half) * 2;
            out[h * vdim + d] = acc[2 * i];
            out[h * vdim + d + 1] = acc[2 * i + 1];
        }
    }
}

// out[b, h, :] = sigmoid(gate[b, h]) * sum over the sequence's runs, in index order; grid (H, B)
template <typename TO>
__global__ void bias_mixed_merge_kernel(const float* __restrict__ part, const int* __restrict__ seq_len, const float* __restrict__ gate,
                                        int ld_gate, TO* __restrict__ out, int H, int vdim, int window, int n_runs) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int len = seq_len[b];
    const int first = bias_first_key(len - 1, window);
    const int rp = bias_run_pages(first, len);
    const int runs = min(n_runs, ((len - 1) / QWB_BIAS_PAGE - first / QWB_BIAS_PAGE) / rp + 1);
    const float gt = gate ? 1.f / (1.f + expf(-gate[(size_t)b * ld_gate + h])) : 1.f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < runs; ++r) a += part[(((size_t)b * n_runs + r) * H + h) * vdim + d];
        out[((size_t)b * H + h) * vdim + d] = from_f32<TO>(a * gt);
    }
}

template <typename T>
static size_t bias_mixed_smem(int H, int G, int dim, int vdim) {
    constexpr int VEC = Vec16<T>::N;
    const int kld = dim + VEC;
    return (size_t)G * QWB_BIAS_PAGE * (kld > vdim ? kld : vdim) * sizeof(T) +
           ((size_t)H * dim + 2 * (size_t)H * QWB_BIAS_PAGE + (size_t)H * H + 3 * (size_t)H) * sizeof(float);
}

// 1 if the two-pass form takes these sizes
extern "C" int qwb_bias_decode_mixed_fits(int dtype, int H, int G, int dim, int vdim) {
    if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || dim % 8 || vdim % 8 || dim > QWB_BIAS_MAX_DIM || vdim > QWB_BIAS_MAX_DIM) return 0;
    if ((long long)H * vdim > (long long)QWB_BIAS_MIXED_THREADS * QWB_BIAS_MIXED_ACC) return 0;
    const size_t smem = dtype == QWB_DT_F32 ? bias_mixed_smem<float>(H, G, dim, vdim) : bias_mixed_smem<bf16>(H, G, dim, vdim);
    return (dtype == QWB_DT_F32 || dtype == QWB_DT_BF16) && smem <= 200 * 1024;
}

// floats of scratch: the first pass's maxima and sums, the heads' stats, the runs' sums
extern "C" long long qwb_bias_decode_mixed_scratch_floats(int B, int H, int vdim, int n_runs) {
    return (long long)B * H * (2 * n_runs + 2) + (long long)B * n_runs * H * vdim;
}

template <typename T>
static int launch_bias_decode_mixed(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                                    float* scratch, void* out, int B, int H, int G, int dim, int vdim, int table_width, float scale,
                                    const float* head_scale, float softcap, const float* slopes, int window, const float* sinks,
                                    const float* mix, const float* gate, int ld_gate, int n_runs, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    float* part_m = scratch;
    float* part_l = part_m + (size_t)B * H * n_runs;
    float* stats = part_l + (size_t)B * H * n_runs;
    float* part = stats + (size_t)B * H * 2;
    const size_t smem1 = ((size_t)QWB_BIAS_PAGE * (dim + VEC) + (size_t)QWB_BIAS_PAGE * vdim) * sizeof(T) +
                         ((size_t)QWB_BIAS_ROWS * dim + QWB_BIAS_ROWS * QWB_BIAS_PAGE + 4 * QWB_BIAS_ROWS) * sizeof(float);
    const size_t smem2 = bias_mixed_smem<T>(H, G, dim, vdim);
    cudaError_t e = cudaSuccess;
    if (smem1 > 48 * 1024) e = cudaFuncSetAttribute(bias_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e == cudaSuccess && smem2 > 48 * 1024) e = cudaFuncSetAttribute(bias_decode_mixed_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "bias_decode_mixed: %s", cudaGetErrorString(e));
    const int slices = (H / G + QWB_BIAS_ROWS - 1) / QWB_BIAS_ROWS;
    qwb_launch(bias_decode_kernel<T>, dim3(n_runs, G * slices, B), 128, smem1, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool,
               page_table, seq_len, (float*)nullptr, part_m, part_l, H, G, 1, dim, vdim, table_width, scale, head_scale, softcap, slopes,
               window, n_runs, 1);
    if (int rc = qwb_check_launch("bias_decode (maxima and sums)")) return rc;
    qwb_launch(bias_stats_kernel, dim3(H, B), 32, 0, stream, (const float*)part_m, (const float*)part_l, seq_len, stats, window, n_runs, sinks);
    if (int rc = qwb_check_launch("bias_stats")) return rc;
    qwb_launch(bias_decode_mixed_kernel<T>, dim3(n_runs, B), QWB_BIAS_MIXED_THREADS, smem2, stream, (const T*)q, (const T*)k_pool,
               (const T*)v_pool, page_table, seq_len, (const float*)stats, mix, part, H, G, dim, vdim, table_width, scale, head_scale,
               softcap, slopes, window, n_runs);
    if (int rc = qwb_check_launch("bias_decode_mixed")) return rc;
    const int block = vdim >= 128 ? 128 : (vdim >= 64 ? 64 : 32);
    qwb_launch(bias_mixed_merge_kernel<T>, dim3(H, B), block, 0, stream, (const float*)part, seq_len, gate, ld_gate, (T*)out, H, vdim,
               window, n_runs);
    return qwb_check_launch("bias_mixed_merge");
}

// q [B, H, dim]; out [B, H * vdim] in the cache's dtype; mix [H, H]; gate: H columns of a float matrix with rows of ld_gate
// values, or null; scratch: qwb_bias_decode_mixed_scratch_floats floats.
extern "C" int qwb_bias_decode_mixed(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                                     float* scratch, void* out, int dtype, int B, int H, int G, int dim, int vdim, int table_width,
                                     float scale, const float* head_scale, float softcap, const float* slopes, int window,
                                     const float* sinks, const float* mix, const float* gate, int ld_gate, int n_runs,
                                     cudaStream_t stream) {
    if (B <= 0) return 0;
    if (int rc = check_bias_sizes("bias_decode_mixed", H, G, dim, vdim, table_width, window, 8)) return rc;
    if (!mix || !qwb_bias_decode_mixed_fits(dtype, H, G, dim, vdim))
        return qwb_fail(QWB_ERR_ARG, "bias_decode_mixed: %d heads over %d, keys of %d and values of %d do not fit this form", H, G, dim, vdim);
    if (n_runs <= 0 || n_runs > 65535 || B > 65535) return qwb_fail(QWB_ERR_ARG, "bias_decode_mixed: %d runs, %d sequences", n_runs, B);
    if (dtype == QWB_DT_F32)
        return launch_bias_decode_mixed<float>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, H, G, dim, vdim, table_width, scale,
                                               head_scale, softcap, slopes, window, sinks, mix, gate, ld_gate, n_runs, stream);
    return launch_bias_decode_mixed<bf16>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, H, G, dim, vdim, table_width, scale,
                                          head_scale, softcap, slopes, window, sinks, mix, gate, ld_gate, n_runs, stream);
}

// ---------------------------------------------------------------------------------
// The mix of the heads after the softmax and the gate:  out[t, h, :] = sigmoid(gate[t, h]) * sum_g M[h, g] a[t, g, c_h, :]
// with c_h = h / (H / G) head h's own value head (C = G), or, without a mix (C = 1), out = sigmoid(gate) * a[t, h, 0, :].
// a [T, H, C, vdim] float; gate: H columns of a float matrix with rows of ld_gate values, or null; grid (T, H).
// ---------------------------------------------------------------------------------
template <typename TO>
__global__ void bias_head_mix_kernel(const float* __restrict__ a, const float* __restrict__ mix, const float* __restrict__ gate,
                                     int ld_gate, TO* __restrict__ out, int H, int G, int C, int vdim) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    const int c = C > 1 ? h / (H / G) : 0;
    const float gt = gate ? 1.f / (1.f + expf(-gate[(size_t)t * ld_gate + h])) : 1.f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float v;
        if (mix) {
            v = 0.f;
            for (int g = 0; g < H; ++g) v += mix[h * H + g] * a[(((size_t)t * H + g) * C + c) * vdim + d];
        } else {
            v = a[(((size_t)t * H + h) * C + c) * vdim + d];
        }
        out[((size_t)t * H + h) * vdim + d] = from_f32<TO>(v * gt);
    }
}

extern "C" int qwb_bias_head_mix(const float* a, const float* mix, const float* gate, int ld_gate, void* out, int out_dtype, int T,
                                 int H, int G, int all_values, int vdim, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || vdim <= 0 || H > 65535) return qwb_fail(QWB_ERR_ARG, "bias_head_mix: %d heads, %d value heads of %d", H, G, vdim);
    if (mix && !all_values) return qwb_fail(QWB_ERR_ARG, "bias_head_mix: a mix of the heads needs every head's output for all value heads");
    const int C = all_values ? G : 1;
    const int block = vdim >= 128 ? 128 : (vdim >= 64 ? 64 : 32);
    if (out_dtype == QWB_DT_F32) qwb_launch(bias_head_mix_kernel<float>, dim3(T, H), block, 0, stream, a, mix, gate, ld_gate, (float*)out, H, G, C, vdim);
    else if (out_dtype == QWB_DT_BF16) qwb_launch(bias_head_mix_kernel<bf16>, dim3(T, H), block, 0, stream, a, mix, gate, ld_gate, (bf16*)out, H, G, C, vdim);
    else return qwb_fail(QWB_ERR_ARG, "bias_head_mix: unknown dtype %d", out_dtype);
    return qwb_check_launch("bias_head_mix");
}
