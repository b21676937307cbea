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
//   bias_decode    one new token per sequence: runs of pages, one block of threads a run, then bias_merge, which also adds
//                  the sink
//   bias_head_mix  the mix of the heads and the gate
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
                                   const float* __restrict__ slopes, int window, int n_runs) {
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
        if (d >= vdim) continue;
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
               n_runs);
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
