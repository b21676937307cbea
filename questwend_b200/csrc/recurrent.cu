// Recurrent mixers: a short causal convolution over time with a tail kept per sequence, the state-space
// recurrence of Mamba-2 and the gated delta rule with one decay per key channel, and the gated norms that
// follow them.  Everything here is 32-bit: inputs are the 32-bit results of the projections, the states are
// float, and so are decays, step sizes, gates and unit norms.
//
// A step brings T packed tokens of B sequences (cu_seqlens [B + 1]); sequence b's state lives in row
// slots[b] of the state tensors.  One token per sequence (a decode step) is the same code with one token.
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

#define QWB_CONV_MAX_TAPS 16

// ---------------------------------------------------------------------------------
// out[t, c] = act( bias[c] + sum_j w[c, j] * in(i - (taps - 1 - j), c) ),  i = the token's index in this step,
// in(i < 0) = the tail: tail[slot, taps - 1 + i, c] (the last taps - 1 inputs of the sequence before this step,
// zero for a new sequence).  x [T, ld] is read at column c (the caller offsets the pointer), out is [T, C].
// in_bias, if given, is added to every input x before it is convolved (a projection's bias: the tail holds inputs with
// it, the zeros before a sequence's start stay zeros).
// act 0: none; 1: SiLU; 2: the token's own input is added to the sum, out = x_t + conv(x)_t.  out is float or bfloat16.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void short_conv_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* __restrict__ in_bias, const float* tail, const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ slots, TOut* __restrict__ out, int T, int C, int taps, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x, t = blockIdx.x;
    if (c >= C || t >= T) return;
    const int b = tok_seq[t];
    const int i = t - cu_seqlens[b];
    float acc = bias ? bias[c] : 0.f;
    const float ib = in_bias ? in_bias[c] : 0.f;
    const float* tl = tail + (size_t)slots[b] * (taps - 1) * C;
    float v = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int src = i - (taps - 1 - j);
        v = src >= 0 ? x[(size_t)(t - (taps - 1 - j)) * ld + c] + ib : tl[(size_t)(taps - 1 + src) * C + c];
        acc += w[c * taps + j] * v;
    }
    out[(size_t)t * C + c] = from_f32<TOut>(act == 1 ? silu_f(acc) : (act == 2 ? acc + v : acc));
}

// The tail after the step: the last taps - 1 inputs of each sequence (new ones, then what is left of the old tail).
__global__ void conv_tail_kernel(const float* __restrict__ x, int ld, const float* __restrict__ in_bias, float* tail,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int B, int C, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C || b >= B) return;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    float* tl = tail + (size_t)slots[b] * (taps - 1) * C;
    float keep[QWB_CONV_MAX_TAPS];
    const float ib = in_bias ? in_bias[c] : 0.f;
    for (int r = 0; r < taps - 1; ++r) {
        const int idx = n_new - (taps - 1) + r;
        keep[r] = idx >= 0 ? x[(size_t)(t0 + idx) * ld + c] + ib : tl[(size_t)(r + n_new) * C + c];
    }
    for (int r = 0; r < taps - 1; ++r) tl[(size_t)r * C + c] = keep[r];
}

// A step of one token per sequence: the convolution and the new tail by one thread per (sequence, channel).
template <typename TOut>
__global__ void short_conv_step_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                                       const float* __restrict__ in_bias, float* tail, const int* __restrict__ slots, TOut* __restrict__ out, int B, int C, int taps,
                                       int act, int update_tail) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x, b = blockIdx.x;
    if (c >= C || b >= B) return;
    float* tl = tail + (size_t)slots[b] * (taps - 1) * C;
    const float cur = x[(size_t)b * ld + c] + (in_bias ? in_bias[c] : 0.f);
    float acc = (bias ? bias[c] : 0.f) + w[c * taps + taps - 1] * cur;
    float keep[QWB_CONV_MAX_TAPS];
    for (int r = 0; r < taps - 1; ++r) {
        keep[r] = tl[(size_t)r * C + c];
        acc += w[c * taps + r] * keep[r];
    }
    out[(size_t)b * C + c] = from_f32<TOut>(act == 1 ? silu_f(acc) : (act == 2 ? acc + cur : acc));
    if (update_tail) {
        for (int r = 0; r + 1 < taps - 1; ++r) tl[(size_t)r * C + c] = keep[r + 1];
        if (taps > 1) tl[(size_t)(taps - 2) * C + c] = cur;
    }
}

template <typename TOut>
static int launch_short_conv(const float* x, int ld, const float* w, const float* bias, const float* in_bias, float* tail, const int* tok_seq,
                             const int* cu_seqlens, const int* slots, TOut* out, int T, int B, int C, int taps, int act,
                             int update_tail, int single_token, cudaStream_t stream) {
    const int block = C >= 256 ? 256 : 128;
    if (single_token && T == B) {
        qwb_launch(short_conv_step_kernel<TOut>, dim3(B, (C + block - 1) / block), block, 0, stream, x, ld, w, bias, in_bias, tail, slots, out, B, C, taps, act, update_tail);
        return qwb_check_launch("short_conv_step");
    }
    qwb_launch(short_conv_kernel<TOut>, dim3(T, (C + block - 1) / block), block, 0, stream, x, ld, w, bias, in_bias, (const float*)tail, tok_seq, cu_seqlens, slots, out, T, C, taps, act);
    if (int rc = qwb_check_launch("short_conv")) return rc;
    if (update_tail && taps > 1) {
        qwb_launch(conv_tail_kernel, dim3((C + block - 1) / block, B), block, 0, stream, x, ld, in_bias, tail, cu_seqlens, slots, B, C, taps);
        return qwb_check_launch("conv_tail");
    }
    return 0;
}

extern "C" int qwb_short_conv(const float* x, int ld, const float* w, const float* bias, const float* in_bias, float* tail, const int* tok_seq,
                              const int* cu_seqlens, const int* slots, void* out, int out_dtype, int T, int B, int C, int taps, int act,
                              int update_tail, int single_token, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > QWB_CONV_MAX_TAPS || ld < C || act < 0 || act > 2)
        return qwb_fail(QWB_ERR_ARG, "short_conv: %d channels, %d taps (1 to %d), row stride %d, mode %d", C, taps, QWB_CONV_MAX_TAPS, ld, act);
    if (B > 65535 || C > 65535 * 128) return qwb_fail(QWB_ERR_ARG, "short_conv: %d sequences or %d channels are too many", B, C);
    if (out_dtype == QWB_DT_F32)
        return launch_short_conv<float>(x, ld, w, bias, in_bias, tail, tok_seq, cu_seqlens, slots, (float*)out, T, B, C, taps, act, update_tail, single_token, stream);
    if (out_dtype == QWB_DT_BF16)
        return launch_short_conv<bf16>(x, ld, w, bias, in_bias, tail, tok_seq, cu_seqlens, slots, (bf16*)out, T, B, C, taps, act, update_tail, single_token, stream);
    return qwb_fail(QWB_ERR_ARG, "short_conv: unknown dtype %d", out_dtype);
}

// ---------------------------------------------------------------------------------
// The recurrences keep, per head, a state matrix S of rows x P (state or key size x value size) whose columns never
// meet: column p is read and written with the token's value p only.  So one WARP owns one column: lane l keeps rows
// l * PER .. l * PER + PER - 1 in registers, a sum over the rows is a shuffle reduction, and there is no shared
// memory and no barrier (a warp takes 2 or 4 columns where few rows fall to a lane: they share the loads of a
// token's vectors); a block is four warps of one head, the grid (warps' columns / 4, heads, sequences).  The state
// is stored column by column, [slots, H, P, rows], so that a warp's piece is one contiguous run.  The vectors of a
// few tokens are asked for together.
// ---------------------------------------------------------------------------------
#define QWB_SCAN_WARPS 4
#define QWB_SCAN_MAX_PER 16

// PER consecutive floats from base[n0 ..], zeros from `limit` on; VEC: n0, limit and base allow 16-byte loads.
template <int PER, bool VEC>
__device__ __forceinline__ void load_rows(const float* __restrict__ base, int n0, int limit, float* out) {
    if (VEC) {
#pragma unroll
        for (int k = 0; k < PER; k += 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (n0 + k < limit) v = *reinterpret_cast<const float4*>(base + n0 + k);
            out[k] = v.x; out[k + 1] = v.y; out[k + 2] = v.z; out[k + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < PER; ++k) out[k] = n0 + k < limit ? base[n0 + k] : 0.f;
    }
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
#define QWB_SCAN_AHEAD 8        // rounds of tokens whose vectors are asked into L2 ahead of their use
#ifndef QWB_SSM_CW_MAX
#define QWB_SSM_CW_MAX 4        // the most columns a warp takes in the Mamba-2 recurrence ...
#endif
#ifndef QWB_DELTA_CW_MAX
#define QWB_DELTA_CW_MAX 2      // ... and in the delta rule (a token's two sums over the rows sit in its chain: 2 measured best)
#endif

// Sums over the warp of 16 values a lane at once: at every step a lane hands half of its values to its partner and adds
// the partner's other half, so the warp needs 8 + 4 + 2 + 1 + 1 shuffles instead of 16 x 5.  Afterwards lane l holds the
// total of value (l >> 1) in v[0] (both lanes of a pair hold it).  The order of the additions is fixed.
__device__ __forceinline__ void warp_sum16(float (&v)[16], int lane) {
#pragma unroll
    for (int half = 8, offset = 16; half >= 1; half >>= 1, offset >>= 1) {
        const bool upper = lane & offset;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float keep = upper ? v[i + half] : v[i];
            const float send = upper ? v[i] : v[i + half];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, offset);
        }
    }
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// Mamba-2.  Per head h (group g = h / (H / G)), per token:
//     dt = softplus(dt_raw + dt_bias[h]);  S = exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x
//   xbc [T, ldx] float: x [H * P] | B [G * N] | C [G * N] (after convolution and SiLU)
//   dt_raw: column h of a [T, ld_dt] matrix;  state [slots, H, P, N];  y [T, H * P]
template <int PER, bool VEC, int TB, int CW>
__global__ void __launch_bounds__(32 * QWB_SCAN_WARPS)
ssm_scan_kernel(const float* __restrict__ xbc, int ldx, const float* __restrict__ dt_raw, int ld_dt,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                float* __restrict__ state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                float* __restrict__ y, int H, int P, int N, int G, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int p0 = (blockIdx.x * QWB_SCAN_WARPS + (threadIdx.x >> 5)) * CW, h = blockIdx.y, b = blockIdx.z;
    if (p0 >= P) return;                                            // P is a multiple of CW: a warp's columns all exist
    const int g = h / (H / G);
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int n0 = lane * PER;
    float* S = state + (((size_t)slots[b] * H + h) * P + p0) * N;
    float s[CW][PER];
#pragma unroll
    for (int c = 0; c < CW; ++c) load_rows<PER, VEC>(S + (size_t)c * N, n0, N, s[c]);
    const float a = -expf(A_log[h]), dskip = Dskip[h], bias = dt_bias[h];
    const int inner = H * P;
    // TB tokens a round: their vectors are asked for together (once for the warp's CW columns) and a round ahead of
    // their use (and into L2 some rounds earlier: a prompt's rows come from HBM once, in the order of the tokens); the
    // state runs through a round's tokens in order, and the sums over the rows are reduced side by side
    float Bn[TB][PER], Cn[TB][PER], dt_n[TB], x_n[TB][CW];
    auto load_round = [&](int tc) {
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const int t = min(tc + j, t1 - 1);                      // past the end: the last token again, not used
            const float* row = xbc + (size_t)t * ldx;
            load_rows<PER, VEC>(row + inner + g * N, n0, N, Bn[j]);
            load_rows<PER, VEC>(row + inner + (G + g) * N, n0, N, Cn[j]);
            dt_n[j] = dt_raw[(size_t)t * ld_dt + h];
#pragma unroll
            for (int c = 0; c < CW; ++c) x_n[j][c] = row[h * P + p0 + c];
        }
    };
    if (t0 < t1) load_round(t0);
    for (int tc = t0; tc < t1; tc += TB) {
        float Bt[TB][PER], Ct[TB][PER], dt_in[TB], xv[TB][CW];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            dt_in[j] = dt_n[j];
#pragma unroll
            for (int k = 0; k < PER; ++k) { Bt[j][k] = Bn[j][k]; Ct[j][k] = Cn[j][k]; }
#pragma unroll
            for (int c = 0; c < CW; ++c) xv[j][c] = x_n[j][c];
        }
        if (tc + TB < t1) load_round(tc + TB);
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const int t = tc + QWB_SCAN_AHEAD * TB + j;
            if (t < t1 && n0 < N) {
                const float* row = xbc + (size_t)t * ldx + inner + g * N + n0;
                prefetch_l2(row);
                prefetch_l2(row + G * N);
                if (lane == 0) prefetch_l2(xbc + (size_t)t * ldx + h * P + p0);
            }
        }
        float acc[TB][CW];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const float dt = softplus_f(dt_in[j] + bias);
            const float decay = expf(a * dt);
#pragma unroll
            for (int c = 0; c < CW; ++c) {
                acc[j][c] = 0.f;
                if (tc + j < t1) {
                    const float dtx = dt * xv[j][c];
#pragma unroll
                    for (int k = 0; k < PER; ++k) {
                        s[c][k] = decay * s[c][k] + dtx * Bt[j][k];
                        acc[j][c] += s[c][k] * Ct[j][k];
                    }
                }
            }
        }
        if (TB * CW == 16) {                                        // the round's 16 sums at once; lane 2 i writes sum i
            float v16[16];
#pragma unroll
            for (int j = 0; j < TB; ++j)
#pragma unroll
                for (int c = 0; c < CW; ++c) v16[(j * CW + c) & 15] = acc[j][c];
            warp_sum16(v16, lane);
            const int mine = lane >> 1, j = mine / CW, c = mine - j * CW;
            float x_mine = 0.f;
#pragma unroll
            for (int jj = 0; jj < TB; ++jj)
#pragma unroll
                for (int cc = 0; cc < CW; ++cc)
                    if (jj * CW + cc == mine) x_mine = xv[jj][cc];
            if (!(lane & 1) && tc + j < t1) y[(size_t)(tc + j) * inner + h * P + p0 + c] = v16[0] + dskip * x_mine;
        } else {
#pragma unroll
            for (int j = 0; j < TB; ++j)
#pragma unroll
                for (int c = 0; c < CW; ++c) acc[j][c] = warp_sum(acc[j][c]);
#pragma unroll
            for (int j = 0; j < TB; ++j)
#pragma unroll
                for (int c = 0; c < CW; ++c)
                    if (lane == 0 && tc + j < t1) y[(size_t)(tc + j) * inner + h * P + p0 + c] = acc[j][c] + dskip * xv[j][c];
        }
    }
    if (write_state) {
#pragma unroll
        for (int c = 0; c < CW; ++c)
#pragma unroll
            for (int k = 0; k < PER; ++k)
                if (n0 + k < N) S[(size_t)c * N + n0 + k] = s[c][k];
    }
}

static int scan_rows_per_lane(int rows) {      // 1, 2, 4, 8 or 16 rows of a column per lane; 0: too many rows
    for (int per = 1; per <= QWB_SCAN_MAX_PER; per *= 2)
        if (32 * per >= rows) return per;
    return 0;
}
static bool aligned16(const void* p) { return (uintptr_t)p % 16 == 0; }

extern "C" int qwb_ssm_scan(const float* xbc, int ldx, const float* dt_raw, int ld_dt, const float* dt_bias, const float* A_log,
                            const float* Dskip, float* state, const int* cu_seqlens, const int* slots, float* y, int B,
                            int H, int P, int N, int G, int write_state, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "ssm_scan: %d heads, %d groups, state %d x %d", H, G, N, P);
    const int per = scan_rows_per_lane(N);
    if (!per) return qwb_fail(QWB_ERR_ARG, "ssm_scan: a state of %d rows per head is too large (up to %d)", N, 32 * QWB_SCAN_MAX_PER);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "ssm_scan: %d sequences or %d heads are too many", B, H);
    const bool vec = per >= 4 && N % 4 == 0 && ldx % 4 == 0 && (H * P) % 4 == 0 && aligned16(xbc) && aligned16(state);
    // columns a warp: 4 or 2 where the rows a lane keeps are few and the value size divides; the columns share the loads
    int cw = per <= 4 && P % 4 == 0 ? 4 : (per <= 8 && P % 2 == 0 ? 2 : 1);
    if (cw > QWB_SSM_CW_MAX) cw = QWB_SSM_CW_MAX;
    const dim3 grid((P / cw + QWB_SCAN_WARPS - 1) / QWB_SCAN_WARPS, H, B);
#define QWB_SSM1(PER, VEC, CW) qwb_launch(ssm_scan_kernel<PER, VEC, (PER <= 4 ? 4 : (PER == 8 ? 2 : 1)), CW>, grid, 32 * QWB_SCAN_WARPS, 0, stream, xbc, ldx, dt_raw, ld_dt, dt_bias, A_log, Dskip, state, cu_seqlens, slots, y, H, P, N, G, write_state)
#define QWB_SSM(PER, VEC) do { if (cw == 4 && PER <= 4) QWB_SSM1(PER, VEC, (PER <= 4 ? 4 : 1)); else if (cw >= 2 && PER <= 8) QWB_SSM1(PER, VEC, (PER <= 8 ? 2 : 1)); else QWB_SSM1(PER, VEC, 1); } while (0)
    if (per == 1) QWB_SSM(1, false); else if (per == 2) QWB_SSM(2, false);
    else if (per == 4) { if (vec) QWB_SSM(4, true); else QWB_SSM(4, false); }
    else if (per == 8) { if (vec) QWB_SSM(8, true); else QWB_SSM(8, false); }
    else { if (vec) QWB_SSM(16, true); else QWB_SSM(16, false); }
#undef QWB_SSM1
#undef QWB_SSM
    return qwb_check_launch("ssm_scan");
}

// ---------------------------------------------------------------------------------
// Gated delta rule, one decay per head and key channel.
// Preparation, one block per token: q and k (after convolution and SiLU) become unit vectors per head,
// x / sqrt(sum x^2 + unit_eps), q times q_scale; kq = k . q; beta = sigmoid(b_raw); decay[h, n] =
// exp(-exp(A_log[h]) softplus(a_raw[h, n] + dt_bias[h, n])).  b_raw: H columns of a matrix with rows of ld_b values.
// decay_k = K: a decay per head and key channel; decay_k = 1: one per head (a_raw then has H columns, in rows of ld_a).
//   qkv [T, ld]: q [Hk * K] | k [Hk * K] | v [H * P], q and k normalised in place
// ---------------------------------------------------------------------------------
__global__ void delta_prep_kernel(float* qkv, int ld, float* __restrict__ kq, const float* __restrict__ b_raw, int ld_b, float* __restrict__ beta,
                                  const float* __restrict__ a_raw, int ld_a, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                  float* __restrict__ decay, int H, int Hk, int K, int decay_k, float unit_eps, float q_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float* row = qkv + (size_t)t * ld;
    for (int kh = warp; kh < Hk; kh += nwarp) {
        float* q = row + kh * K;
        float* k = row + (Hk + kh) * K;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < K; i += 32) { sq += q[i] * q[i]; sk += k[i] * k[i]; }
        sq = warp_sum(sq); sk = warp_sum(sk);
        const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.f / sqrtf(sk + unit_eps);
        float dot = 0.f;
        for (int i = lane; i < K; i += 32) {
            const float qn = q[i] * rq, kn = k[i] * rk;
            q[i] = qn; k[i] = kn;
            dot += qn * kn;
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(size_t)t * Hk + kh] = dot;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) beta[(size_t)t * H + i] = sigmoid_f(b_raw[(size_t)t * ld_b + i]);
    for (int i = threadIdx.x; i < H * decay_k; i += blockDim.x)
        decay[(size_t)t * H * decay_k + i] = expf(-expf(A_log[i / decay_k]) * softplus_f(a_raw[(size_t)t * ld_a + i] + dt_bias[i]));
}

extern "C" int qwb_delta_prep(float* qkv, int ld, float* kq, const float* b_raw, int ld_b, float* beta, const float* a_raw, int ld_a,
                              const float* dt_bias, const float* A_log, float* decay, int T, int H, int Hk, int K, int decay_k,
                              float unit_eps, float q_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Hk <= 0 || K <= 0 || H % Hk) return qwb_fail(QWB_ERR_ARG, "delta_prep: %d heads, %d key heads of %d", H, Hk, K);
    if ((decay_k != K && decay_k != 1) || ld_a < H * decay_k) return qwb_fail(QWB_ERR_ARG, "delta_prep: %d decays a head (1 or %d) in rows of %d", decay_k, K, ld_a);
    qwb_launch(delta_prep_kernel, T, 128, 0, stream, qkv, ld, kq, b_raw, ld_b, beta, a_raw, ld_a, dt_bias, A_log, decay, H, Hk, K, decay_k, unit_eps, q_scale);
    return qwb_check_launch("delta_prep");
}

// Preparation for gated linear attention, one block per token: q times q_scale in place, kq = k . q per head, and the
// decay per head and key channel, decay = sigmoid(a_raw + a_bias)^(1 / tau), formed as exp(log_sigmoid(z) / tau) with
// log_sigmoid(z) = -softplus(-z).  qkv [T, ld]: q [H * K] | k [H * K] | v.
__global__ void gla_prep_kernel(float* qkv, int ld, float* __restrict__ kq, const float* __restrict__ a_raw, const float* __restrict__ a_bias,
                                float* __restrict__ decay, int H, int K, float q_scale, float inv_tau) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float* row = qkv + (size_t)t * ld;
    for (int h = warp; h < H; h += nwarp) {
        float* q = row + h * K;
        const float* k = row + (H + h) * K;
        float dot = 0.f;
        for (int i = lane; i < K; i += 32) {
            const float qs = q[i] * q_scale;
            q[i] = qs;
            dot += qs * k[i];
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(size_t)t * H + h] = dot;
    }
    for (int i = threadIdx.x; i < H * K; i += blockDim.x)
        decay[(size_t)t * H * K + i] = expf(-softplus_f(-(a_raw[(size_t)t * H * K + i] + (a_bias ? a_bias[i] : 0.f))) * inv_tau);
}

extern "C" int qwb_gla_prep(float* qkv, int ld, float* kq, const float* a_raw, const float* a_bias, float* decay, int T, int H, int K,
                            float q_scale, float tau, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || !(tau > 0.f)) return qwb_fail(QWB_ERR_ARG, "gla_prep: %d heads of %d, tau %g", H, K, (double)tau);
    qwb_launch(gla_prep_kernel, T, 128, 0, stream, qkv, ld, kq, a_raw, a_bias, decay, H, K, q_scale, 1.f / tau);
    return qwb_check_launch("gla_prep");
}

// Preparation for linear attention with positions, one block per token: the first rdims values of every head of q and k
// are turned (value i with value i + rdims / 2) by the token's angles (cos_t, sin_t [T, rdims / 2]; rdims 0: no turn), then
// q times q_scale and k times k_scale in place, and kq = k . q per head.  qkv [T, ld]: q [H * K] | k [H * K] | v.
__global__ void turn_qk_prep_kernel(float* qkv, int ld, float* __restrict__ kq, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    int H, int K, int rdims, float q_scale, float k_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int half = rdims >> 1;
    float* row = qkv + (size_t)t * ld;
    const float* cs = cos_t + (size_t)t * half;
    const float* sn = sin_t + (size_t)t * half;
    for (int h = warp; h < H; h += nwarp) {
        float* q = row + h * K;
        float* k = row + (H + h) * K;
        float dot = 0.f;
        for (int i = lane; i < half; i += 32) {
            const float c = cs[i], s = sn[i];
            const float qa = q[i], qb = q[i + half], ka = k[i], kb = k[i + half];
            const float q0 = (qa * c - qb * s) * q_scale, q1 = (qb * c + qa * s) * q_scale;
            const float k0 = (ka * c - kb * s) * k_scale, k1 = (kb * c + ka * s) * k_scale;
            q[i] = q0; q[i + half] = q1; k[i] = k0; k[i + half] = k1;
            dot += q0 * k0 + q1 * k1;
        }
        for (int i = rdims + lane; i < K; i += 32) {
            const float qv = q[i] * q_scale, kv = k[i] * k_scale;
            q[i] = qv; k[i] = kv;
            dot += qv * kv;
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(size_t)t * H + h] = dot;
    }
}

extern "C" int qwb_turn_qk_prep(float* qkv, int ld, float* kq, const float* cos_t, const float* sin_t, int T, int H, int K, int rdims,
                                float q_scale, float k_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || rdims < 0 || rdims > K || rdims % 2 || ld < 2 * H * K)
        return qwb_fail(QWB_ERR_ARG, "turn_qk_prep: %d heads of %d, %d turned, rows of %d", H, K, rdims, ld);
    if (rdims > 0 && (!cos_t || !sin_t)) return qwb_fail(QWB_ERR_ARG, "turn_qk_prep: a rotation without its table");
    qwb_launch(turn_qk_prep_kernel, T, 128, 0, stream, qkv, ld, kq, cos_t, sin_t, H, K, rdims, q_scale, k_scale);
    return qwb_check_launch("turn_qk_prep");
}

// The recurrence, per head h (key head kh = h / (H / Hk)), per token, S is K x P:
//     S = decay[:, None] * S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q
// o is formed as (decayed S)^T q + u (k . q), so that both sums over the rows are taken in one pass.  A warp per
// column, as above; state [slots, H, P, K].  Without `beta` (null) the write is the plain outer product, u = v: gated
// linear attention, S = decay[:, None] * S + k v^T.  The decays of token t, head h: decay_k = K values at decay +
// t * decay_ts + h * K (one per key channel), or decay_k = 1 value at decay + t * decay_ts + h (one per head; with
// decay_ts = 0 the same H numbers for every token: a fixed decay per head).
template <int PER, bool VEC, int TB, int CW, bool PC>     // PC: a decay per key channel (else one per head)
__global__ void __launch_bounds__(32 * QWB_SCAN_WARPS)
delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ kq, const float* __restrict__ beta,
                  const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int Hk, int K, int P, int write_state,
                  int decay_ts, int decay_k) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int p0 = (blockIdx.x * QWB_SCAN_WARPS + (threadIdx.x >> 5)) * CW, h = blockIdx.y, b = blockIdx.z;
    if (p0 >= P) return;                                            // P is a multiple of CW: a warp's columns all exist
    const int kh = h / (H / Hk);
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int n0 = lane * PER;
    float* S = state + (((size_t)slots[b] * H + h) * P + p0) * K;
    float s[CW][PER];
#pragma unroll
    for (int c = 0; c < CW; ++c) load_rows<PER, VEC>(S + (size_t)c * K, n0, K, s[c]);
    const int v_at = 2 * Hk * K + h * P + p0;
    // TB tokens a round: their vectors are asked for together (once for the warp's CW columns) and a round ahead of
    // their use (and into L2 some rounds earlier); the state then runs through a round's tokens in order (a token's
    // write needs the sum over the rows of the token before it), the columns side by side
    float kn[TB][PER], qn[TB][PER], gn[TB][PC ? PER : 1], v_n[TB][CW], bt_n[TB], kq_n[TB];
    auto load_round = [&](int tc) {
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const int t = min(tc + j, t1 - 1);                      // past the end: the last token again, not used
            const float* row = qkv + (size_t)t * ld;
            load_rows<PER, VEC>(row + kh * K, n0, K, qn[j]);
            load_rows<PER, VEC>(row + (Hk + kh) * K, n0, K, kn[j]);
            if (PC) load_rows<PC ? PER : 1, PC && VEC>(decay + (size_t)t * decay_ts + h * K, n0, K, gn[j]);
            else gn[j][0] = decay[(size_t)t * decay_ts + h];
#pragma unroll
            for (int c = 0; c < CW; ++c) v_n[j][c] = row[v_at + c];
            bt_n[j] = beta ? beta[(size_t)t * H + h] : 0.f; kq_n[j] = kq[(size_t)t * Hk + kh];
        }
    };
    if (t0 < t1) load_round(t0);
    for (int tc = t0; tc < t1; tc += TB) {
        float kk[TB][PER], qq[TB][PER], gg[TB][PC ? PER : 1], v[TB][CW], bt[TB], kqv[TB];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            bt[j] = bt_n[j]; kqv[j] = kq_n[j];
#pragma unroll
            for (int k = 0; k < PER; ++k) { kk[j][k] = kn[j][k]; qq[j][k] = qn[j][k]; }
#pragma unroll
            for (int k = 0; k < (PC ? PER : 1); ++k) gg[j][k] = gn[j][k];
#pragma unroll
            for (int c = 0; c < CW; ++c) v[j][c] = v_n[j][c];
        }
        if (tc + TB < t1) load_round(tc + TB);
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const int t = tc + QWB_SCAN_AHEAD * TB + j;
            if (t < t1 && n0 < K) {
                const float* row = qkv + (size_t)t * ld;
                prefetch_l2(row + kh * K + n0);
                prefetch_l2(row + (Hk + kh) * K + n0);
                if (PC) prefetch_l2(decay + (size_t)t * decay_ts + h * K + n0);
                if (lane == 0) prefetch_l2(row + v_at);
            }
        }
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            if (tc + j < t1) {
                float sk[CW], sq[CW];
#pragma unroll
                for (int c = 0; c < CW; ++c) {
                    sk[c] = sq[c] = 0.f;
#pragma unroll
                    for (int k = 0; k < PER; ++k) {
                        s[c][k] *= gg[j][PC ? k : 0];
                        sk[c] += s[c][k] * kk[j][k];
                        sq[c] += s[c][k] * qq[j][k];
                    }
                }
#pragma unroll
                for (int c = 0; c < CW; ++c) { sk[c] = warp_sum(sk[c]); sq[c] = warp_sum(sq[c]); }
#pragma unroll
                for (int c = 0; c < CW; ++c) {
                    const float u = beta ? bt[j] * (v[j][c] - sk[c]) : v[j][c];
#pragma unroll
                    for (int k = 0; k < PER; ++k) s[c][k] += kk[j][k] * u;
                    if (lane == 0) o[((size_t)(tc + j) * H + h) * P + p0 + c] = sq[c] + u * kqv[j];
                }
            }
        }
    }
    if (write_state) {
#pragma unroll
        for (int c = 0; c < CW; ++c)
#pragma unroll
            for (int k = 0; k < PER; ++k)
                if (n0 + k < K) S[(size_t)c * K + n0 + k] = s[c][k];
    }
}

extern "C" int qwb_delta_scan(const float* qkv, int ld, const float* kq, const float* beta, const float* decay, float* state,
                              const int* cu_seqlens, const int* slots, float* o, int B, int H, int Hk, int K, int P,
                              int write_state, int decay_ts, int decay_k, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || Hk <= 0 || K <= 0 || P <= 0 || H % Hk) return qwb_fail(QWB_ERR_ARG, "delta_scan: %d heads, %d key heads, state %d x %d", H, Hk, K, P);
    if ((decay_k != K && decay_k != 1) || decay_ts < 0 || (decay_ts != 0 && decay_ts < H * decay_k))
        return qwb_fail(QWB_ERR_ARG, "delta_scan: %d decays a head (1 or %d), %d a token", decay_k, K, decay_ts);
    const int per = scan_rows_per_lane(K);
    if (!per) return qwb_fail(QWB_ERR_ARG, "delta_scan: a state of %d rows per head is too large (up to %d)", K, 32 * QWB_SCAN_MAX_PER);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "delta_scan: %d sequences or %d heads are too many", B, H);
    const bool vec = per >= 4 && K % 4 == 0 && ld % 4 == 0 && aligned16(qkv) && aligned16(state) &&
                     (decay_k != K || (aligned16(decay) && decay_ts % 4 == 0));
    int cw = per <= 4 && P % 4 == 0 ? 4 : (per <= 8 && P % 2 == 0 ? 2 : 1);            // columns a warp, as in ssm_scan
    if (cw > QWB_DELTA_CW_MAX) cw = QWB_DELTA_CW_MAX;
    const dim3 grid((P / cw + QWB_SCAN_WARPS - 1) / QWB_SCAN_WARPS, H, B);
    const bool pc = decay_k > 1 || K == 1;
#define QWB_DELTA0(PER, VEC, CW, PC) qwb_launch(delta_scan_kernel<PER, VEC, (PER <= 4 ? 4 : (PER == 8 ? 2 : 1)), CW, PC>, grid, 32 * QWB_SCAN_WARPS, 0, stream, qkv, ld, kq, beta, decay, state, cu_seqlens, slots, o, H, Hk, K, P, write_state, decay_ts, decay_k)
#define QWB_DELTA1(PER, VEC, CW) do { if (pc) QWB_DELTA0(PER, VEC, CW, true); else QWB_DELTA0(PER, VEC, CW, false); } while (0)
#define QWB_DELTA(PER, VEC) do { if (cw == 4 && PER <= 4) QWB_DELTA1(PER, VEC, (PER <= 4 ? 4 : 1)); else if (cw >= 2 && PER <= 8) QWB_DELTA1(PER, VEC, (PER <= 8 ? 2 : 1)); else QWB_DELTA1(PER, VEC, 1); } while (0)
    if (per == 1) QWB_DELTA(1, false); else if (per == 2) QWB_DELTA(2, false);
    else if (per == 4) { if (vec) QWB_DELTA(4, true); else QWB_DELTA(4, false); }
    else if (per == 8) { if (vec) QWB_DELTA(8, true); else QWB_DELTA(8, false); }
    else { if (vec) QWB_DELTA(16, true); else QWB_DELTA(16, false); }
#undef QWB_DELTA0
#undef QWB_DELTA1
#undef QWB_DELTA
    return qwb_check_launch("delta_scan");
}

// ---------------------------------------------------------------------------------
// Linear attention with a FIXED decay per head over long prompts, in chunks of 64 tokens.  The recurrence
// S <- d S + k v^T, o = S^T q is linear in S, so with S0 the state at a chunk's start and i, j tokens of the chunk
//     o_i = d^(i+1) S0^T q_i + sum_{j <= i} d^(i-j) (q_i . k_j) v_j,      S_end = d^n S0 + sum_j d^(n-1-j) k_j v_j^T
// and chunks compose exactly up to rounding.  Three kernels, all 32-bit: every chunk's own sum of outer products from
// a zero state (chunk_state), the carries through a sequence's chunks in order, which leave each chunk's S0 in the
// scratch and the final state in the cache (chunk_carry), and the chunks' outputs (chunk_out).  A chunk is a block, so
// a prompt of 2,048 tokens and 16 heads is 512 blocks instead of a chain of 2,048 steps.  The powers of d are made in
// 64-bit.  qkv [T, ld]: q [H * K] | k [H * K] | v [H * P], already turned and scaled; scratch [2, B * chunks, H, P, K].
// ---------------------------------------------------------------------------------
#define QWB_CHUNK 64

// 16 bytes from global to shared memory without a register in between: a block's loads are all in flight at once
__device__ __forceinline__ void chunk_cp16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void chunk_cp_wait() {
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// d^n for a small whole n, in 64-bit, by squaring (a dozen multiplications; the library's pow is a long routine)
__device__ __forceinline__ double chunk_pow(double d, int n) {
    double r = 1.0;
    for (; n > 0; n >>= 1, d *= d)
        if (n & 1) r *= d;
    return r;
}

// grid (chunks, H, B), 256 threads; dynamic shared memory: QWB_CHUNK * (K + P + 1) floats
__global__ void __launch_bounds__(256)
retention_chunk_state_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                             float* __restrict__ scratch, int H, int K, int P, int n_chunks) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float cs_smem[];
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = cu_seqlens[b] + c * QWB_CHUNK, t1 = min(cu_seqlens[b + 1], t0 + QWB_CHUNK);
    if (t0 >= t1) return;
    const int n = t1 - t0;
    float* ks = cs_smem;                    // [n][K]
    float* vs = ks + QWB_CHUNK * K;         // [n][P], times d^(n - 1 - j)
    float* pw = vs + QWB_CHUNK * P;         // [QWB_CHUNK] powers of the decay
    const double d = (double)decay[h];
    const int K4c = K >> 2, P4c = P >> 2;
    for (int idx = threadIdx.x; idx < n * K4c; idx += blockDim.x) {
        const int j = idx / K4c, k = (idx - j * K4c) * 4;
        chunk_cp16(ks + j * K + k, qkv + (size_t)(t0 + j) * ld + (H + h) * K + k);
    }
    for (int idx = threadIdx.x; idx < n * P4c; idx += blockDim.x) {
        const int j = idx / P4c, p = (idx - j * P4c) * 4;
        chunk_cp16(vs + j * P + p, qkv + (size_t)(t0 + j) * ld + 2 * H * K + h * P + p);
    }
    for (int i = threadIdx.x; i < QWB_CHUNK; i += blockDim.x) pw[i] = (float)chunk_pow(d, i);
    chunk_cp_wait();
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * P; idx += blockDim.x) vs[idx] *= pw[n - 1 - idx / P];
    __syncthreads();
    float* U = scratch + (((size_t)b * n_chunks + c) * H + h) * (size_t)P * K;
    const int K4 = K >> 2;
    {                                                               // 4 value columns x 4 key rows a thread
        for (int idx = threadIdx.x; idx < (P >> 2) * K4; idx += blockDim.x) {
            const int p4 = idx / K4, k4 = idx - p4 * K4;
            float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll 4
            for (int j = 0; j < n; ++j) {
                const float4 kk = *reinterpret_cast<const float4*>(ks + j * K + 4 * k4);
                const float4 vv = *reinterpret_cast<const float4*>(vs + j * P + 4 * p4);
                a0.x += kk.x * vv.x; a0.y += kk.y * vv.x; a0.z += kk.z * vv.x; a0.w += kk.w * vv.x;
                a1.x += kk.x * vv.y; a1.y += kk.y * vv.y; a1.z += kk.z * vv.y; a1.w += kk.w * vv.y;
                a2.x += kk.x * vv.z; a2.y += kk.y * vv.z; a2.z += kk.z * vv.z; a2.w += kk.w * vv.z;
                a3.x += kk.x * vv.w; a3.y += kk.y * vv.w; a3.z += kk.z * vv.w; a3.w += kk.w * vv.w;
            }
            float* u = U + (size_t)(4 * p4) * K + 4 * k4;
            *reinterpret_cast<float4*>(u) = a0;
            *reinterpret_cast<float4*>(u + K) = a1;
            *reinterpret_cast<float4*>(u + 2 * K) = a2;
            *reinterpret_cast<float4*>(u + 3 * K) = a3;
        }
    }
}

// grid (ceil(P * K / 256), H, B): every element of the state runs through its sequence's chunks in order
__global__ void retention_chunk_carry_kernel(const float* __restrict__ decay, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                             float* __restrict__ state, const float* __restrict__ sums, float* __restrict__ starts,
                                             int H, int K, int P, int n_chunks, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, b = blockIdx.z;
    if (e >= P * K) return;
    const int n_tok = cu_seqlens[b + 1] - cu_seqlens[b];
    if (n_tok <= 0) return;
    const double d = (double)decay[h];
    const float d_full = (float)chunk_pow(d, QWB_CHUNK);
    float* S = state + ((size_t)slots[b] * H + h) * (size_t)P * K + e;
    float s = *S;
    const int chunks = (n_tok + QWB_CHUNK - 1) / QWB_CHUNK;
    const int last = n_tok - (chunks - 1) * QWB_CHUNK;
    const float d_last = last == QWB_CHUNK ? d_full : (float)chunk_pow(d, last);
    const size_t stride = (size_t)H * P * K, at = ((size_t)b * n_chunks * H + h) * (size_t)P * K + e;
#pragma unroll 4
    for (int c = 0; c < chunks; ++c) {
        const float own = sums[at + c * stride];
        starts[at + c * stride] = s;                                // the state this chunk starts from
        s = (c + 1 < chunks ? d_full : d_last) * s + own;
    }
    if (write_state) *S = s;
}

// grid (chunks, H, B), 256 threads; dynamic shared memory: see retention_chunk_smem_floats
__global__ void __launch_bounds__(256)
retention_chunk_out_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                           const float* __restrict__ scratch, float* __restrict__ o, int H, int K, int P, int n_chunks) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int L = QWB_CHUNK, IB = 8;
    extern __shared__ __align__(16) float co_smem[];
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = cu_seqlens[b] + c * L, t1 = min(cu_seqlens[b + 1], t0 + L);
    if (t0 >= t1) return;
    const int n = t1 - t0, KP = K > P ? K : P;
    float* qs = co_smem;                    // [L][K]
    float* kv = qs + L * K;                 // the keys [L][K + 4] (rows 16 bytes off a multiple of 128), then the values [L][P]
    float* A = kv + L * (KP + 4);           // [L][L + 1]
    float* S0 = A + L * (L + 1);            // [P][K + 4]: rows that start 16 bytes off a multiple of 128, read 16 bytes at a time
    float* pw = S0 + (size_t)P * (K + 4);   // [L + 1] powers of the decay
    const double d = (double)decay[h];
    const int K4c = K >> 2, P4c = P >> 2;
    for (int idx = threadIdx.x; idx < n * K4c; idx += blockDim.x) {
        const int j = idx / K4c, k = (idx - j * K4c) * 4;
        const float* row = qkv + (size_t)(t0 + j) * ld;
        chunk_cp16(qs + j * K + k, row + h * K + k);
        chunk_cp16(kv + j * (K + 4) + k, row + (H + h) * K + k);
    }
    const float* S = scratch + (((size_t)b * n_chunks + c) * H + h) * (size_t)P * K;
    for (int idx = threadIdx.x; idx < P * K4c; idx += blockDim.x) {
        const int p = idx / K4c, k = (idx - p * K4c) * 4;
        chunk_cp16(S0 + p * (K + 4) + k, S + (size_t)p * K + k);
    }
    for (int i = threadIdx.x; i <= L; i += blockDim.x) pw[i] = (float)chunk_pow(d, i);
    chunk_cp_wait();
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * n; idx += blockDim.x) {      // A[i][j] = d^(i - j) q_i . k_j for j <= i
        const int i = idx / n, j = idx - i * n;
        float dot = 0.f;
        if (j <= i) {
            const float4* qa = reinterpret_cast<const float4*>(qs + i * K);
            const float4* kb = reinterpret_cast<const float4*>(kv + j * (K + 4));
            for (int k = 0; k < (K >> 2); ++k) {
                const float4 x = qa[k], y = kb[k];
                dot += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
            }
            dot *= pw[i - j];
        }
        A[i * (L + 1) + j] = dot;
    }
    __syncthreads();                                                    // the keys are no longer read
    for (int idx = threadIdx.x; idx < n * P4c; idx += blockDim.x) {
        const int j = idx / P4c, p = (idx - j * P4c) * 4;
        chunk_cp16(kv + j * P + p, qkv + (size_t)(t0 + j) * ld + 2 * H * K + h * P + p);
    }
    chunk_cp_wait();
    __syncthreads();
    const int groups = (n + IB - 1) / IB;
    for (int idx = threadIdx.x; idx < groups * P; idx += blockDim.x) {  // IB tokens of one value column a thread
        const int ig = idx / P, p = idx - ig * P, i0 = ig * IB;
        float acc[IB];
#pragma unroll
        for (int ii = 0; ii < IB; ++ii) acc[ii] = 0.f;
        const float4* srow = reinterpret_cast<const float4*>(S0 + p * (K + 4));
        const float4* qrow[IB];
#pragma unroll
        for (int ii = 0; ii < IB; ++ii) qrow[ii] = reinterpret_cast<const float4*>(qs + min(i0 + ii, n - 1) * K);
        for (int k = 0; k < (K >> 2); ++k) {
            const float4 sv = srow[k];
#pragma unroll
            for (int ii = 0; ii < IB; ++ii) {
                const float4 qv = qrow[ii][k];
                acc[ii] += sv.x * qv.x + sv.y * qv.y + sv.z * qv.z + sv.w * qv.w;
            }
        }
#pragma unroll
        for (int ii = 0; ii < IB; ++ii) acc[ii] *= pw[min(i0 + ii, n - 1) + 1];
        const int j_end = min(i0 + IB, n);
        for (int j = 0; j < j_end; ++j) {
            const float v = kv[j * P + p];
#pragma unroll
            for (int ii = 0; ii < IB; ++ii) acc[ii] += A[min(i0 + ii, n - 1) * (L + 1) + j] * v;      // zero for j > i
        }
#pragma unroll
        for (int ii = 0; ii < IB; ++ii)
            if (i0 + ii < n) o[((size_t)(t0 + i0 + ii) * H + h) * P + p] = acc[ii];
    }
}

static size_t retention_chunk_smem_floats(int K, int P) {
    const int KP = K > P ? K : P;
    return (size_t)QWB_CHUNK * K + (size_t)QWB_CHUNK * (KP + 4) + (size_t)QWB_CHUNK * (QWB_CHUNK + 1) + (size_t)P * (K + 4) + QWB_CHUNK + 1;
}

// 1 if the chunked form takes these sizes (keys and values in multiples of 4, tiles that fit in shared memory)
extern "C" int qwb_retention_chunked_fits(int K, int P) {
    return K > 0 && P > 0 && K % 4 == 0 && P % 4 == 0 && retention_chunk_smem_floats(K, P) * sizeof(float) <= 200 * 1024;
}

extern "C" int qwb_retention_chunk_len() { return QWB_CHUNK; }

// scratch: 2 * B * ceil(max_new / 64) * H * P * K floats (the chunks' own sums, then the states they start from)
extern "C" int qwb_retention_chunked(const float* qkv, int ld, const float* decay, float* state, const int* cu_seqlens, const int* slots,
                                     float* scratch, float* o, int B, int max_new, int H, int K, int P, int write_state, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (H <= 0 || !qwb_retention_chunked_fits(K, P) || ld < H * (2 * K + P) || ld % 4 || (uintptr_t)qkv % 16 || (uintptr_t)scratch % 16)
        return qwb_fail(QWB_ERR_ARG, "retention_chunked: %d heads of %d x %d in rows of %d", H, K, P, ld);
    const int n_chunks = (max_new + QWB_CHUNK - 1) / QWB_CHUNK;
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "retention_chunked: %d sequences or %d heads are too many", B, H);
    const size_t smem1 = (size_t)QWB_CHUNK * (K + P + 1) * sizeof(float), smem3 = retention_chunk_smem_floats(K, P) * sizeof(float);
    cudaError_t e = cudaSuccess;
    if (smem1 > 48 * 1024) e = cudaFuncSetAttribute(retention_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e == cudaSuccess && smem3 > 48 * 1024) e = cudaFuncSetAttribute(retention_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "retention_chunked: %s", cudaGetErrorString(e));
    qwb_launch(retention_chunk_state_kernel, dim3(n_chunks, H, B), 256, smem1, stream, qkv, ld, decay, cu_seqlens, scratch, H, K, P, n_chunks);
    if (int rc = qwb_check_launch("retention_chunk_state")) return rc;
    float* starts = scratch + (size_t)B * n_chunks * H * P * K;
    qwb_launch(retention_chunk_carry_kernel, dim3((P * K + 255) / 256, H, B), 256, 0, stream, decay, cu_seqlens, slots, state, (const float*)scratch, starts, H, K, P, n_chunks, write_state);
    if (int rc = qwb_check_launch("retention_chunk_carry")) return rc;
    qwb_launch(retention_chunk_out_kernel, dim3(n_chunks, H, B), 256, smem3, stream, qkv, ld, decay, cu_seqlens, (const float*)starts, o, H, K, P, n_chunks);
    return qwb_check_launch("retention_chunk_out");
}

// ---------------------------------------------------------------------------------
// Gated norm over equal parts of a row.  y [T, n_parts * part] float, gate: column slice of a [T, ld_gate] matrix.
//   mode 0: v = y * silu(gate); out = v / rms(v over the part) * w      (the gate before the norm)
//   mode 1: out = y / rms(y over the part) * w * sigmoid(gate)          (the gate after the norm)
//   mode 2: out = y / rms(y over the part) * w * silu(gate)
// w has w_len entries and is indexed by column % w_len (the whole row, or one part shared by all parts).
// One warp per (token, part).
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void gated_part_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate,
                                       const float* __restrict__ w, int w_len, TOut* __restrict__ out, int T, int n_parts,
                                       int part, float eps, int mode) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)T * n_parts) return;
    const int t = (int)(unit / n_parts), g = (int)(unit % n_parts);
    const int D = n_parts * part;
    const float* yr = y + (size_t)t * D + g * part;
    const float* gr = gate + (size_t)t * ld_gate + g * part;
    float ss = 0.f;
    for (int i = lane; i < part; i += 32) {
        const float v = mode == 0 ? yr[i] * silu_f(gr[i]) : yr[i];
        ss += v * v;
    }
    const float scale = rsqrtf(warp_sum(ss) / (float)part + eps);
    TOut* orow = out + (size_t)t * D + g * part;
    for (int i = lane; i < part; i += 32) {
        const float wi = w[(g * part + i) % w_len];
        const float v = mode == 0 ? yr[i] * silu_f(gr[i]) * scale * wi : yr[i] * scale * wi * (mode == 1 ? sigmoid_f(gr[i]) : silu_f(gr[i]));
        orow[i] = from_f32<TOut>(v);
    }
}

extern "C" int qwb_gated_part_norm(const float* y, const float* gate, int ld_gate, const float* w, int w_len, void* out,
                                   int out_dtype, int T, int n_parts, int part, float eps, int mode, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_parts <= 0 || part <= 0 || w_len <= 0 || mode < 0 || mode > 2)
        return qwb_fail(QWB_ERR_ARG, "gated_part_norm: %d parts of %d, weight of %d, mode %d", n_parts, part, w_len, mode);
    const long long units = (long long)T * n_parts;
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (out_dtype == QWB_DT_F32)
        qwb_launch(gated_part_norm_kernel<float>, blocks, 128, 0, stream, y, gate, ld_gate, w, w_len, (float*)out, T, n_parts, part, eps, mode);
    else if (out_dtype == QWB_DT_BF16)
        qwb_launch(gated_part_norm_kernel<bf16>, blocks, 128, 0, stream, y, gate, ld_gate, w, w_len, (bf16*)out, T, n_parts, part, eps, mode);
    else
        return qwb_fail(QWB_ERR_ARG, "gated_part_norm: unknown dtype %d", out_dtype);
    return qwb_check_launch("gated_part_norm");
}
