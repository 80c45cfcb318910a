// The gated delta rule: a matrix memory per head that is decayed, corrected towards the new value and read, token by token.
//
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S: [d, dv] per (request, head), float
//   beta_t = sigmoid(b_t),   g_t = exp(-exp(A_log) softplus(a_t + dt_bias))                 b_t, a_t: two small projections
//
// q, k, v first pass a short causal convolution over time per channel and silu; q and k are then scaled to unit length per
// head (x / sqrt(sum x^2 + unit_eps)), q also by q_scale.  Several value heads may share a q/k head.  Three kernels:
//   conv_prep     convolution (the `taps - 1` inputs before the step come from the request's slot), silu, unit length
//   conv_keep     the slot's last `taps - 1` inputs after the step
//   delta_scan    the recurrence; a thread owns R consecutive rows of one value column of S in registers, IS threads a
//                 column, 16 columns a block; the two column sums a token needs are finished by shuffles.
// Everything is float: the convolution's sums, the unit norms, gates, decays and the state.  The sequence of operations on a
// state element and on an output does not depend on where a step was cut.
#include "common.cuh"

constexpr int DELTA_JS = 16;     // value columns a block
constexpr int DELTA_C = 16;      // tokens a chunk
constexpr int DELTA_TOK = 4;     // tokens a warp of conv_prep takes one after the other
constexpr int CONV_KEEP = 8;     // values of a head a lane keeps in registers (heads of up to 256)

// ------------------------------------------------------------------ convolution + silu + unit length
// grid (requests, chunks of DELTA_TOK tokens, units / 4); a warp a unit (a head of q, k or v) of the chunk's tokens: a token's
// taps reach back into rows the warp has just read.  Output float [T, C].
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) conv_prep_kernel(const TA* __restrict__ proj, int stride, const TW* __restrict__ taps_w, int taps,
                                                        const float* __restrict__ conv_state, long long slot_stride,
                                                        const int* __restrict__ q_start, const int* __restrict__ slots,
                                                        float* __restrict__ out, int C, int nqk, int d, int nv, int dv,
                                                        float unit_eps, float q_scale) {
    const int b = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const int c0 = t0 + blockIdx.y * DELTA_TOK, c1 = min(t1, c0 + DELTA_TOK);
    if (c0 >= t1) return;
    const float* st = conv_state + (size_t)slots[b] * slot_stride;       // [taps - 1][C], oldest first
    const int u = blockIdx.z * 4 + wid;                                  // a warp a unit, the chunk's tokens one after the other
    if (u >= 2 * nqk + nv) return;
    for (int t = c0; t < c1; ++t) {
        const bool qk = u < 2 * nqk;
        const int width = qk ? d : dv, base = qk ? u * d : 2 * nqk * d + (u - 2 * nqk) * dv;
        const int i = t - t0;                                            // the token's place in the step
        const float unit_scale = u < nqk ? q_scale : 1.0f;
        auto conv_at = [&](int c) {                                      // convolution and silu of channel c at this token
            float acc = 0.f;
            for (int j = 0; j < taps; ++j) {                             // tap j reads the input taps - 1 - j tokens back
                const int back = taps - 1 - j, src = i - back;
                const float xin = src >= 0 ? to_f<TA>(proj[(size_t)(t0 + src) * stride + c])
                                           : st[(size_t)(taps - 1 + src) * C + c];
                acc = fmaf(to_f<TW>(taps_w[(size_t)c * taps + j]), xin, acc);
            }
            return acc / (1.0f + expf(-acc));
        };
        if (width <= 32 * CONV_KEEP) {                                   // a head's values stay in registers until its length is known
            float y[CONV_KEEP];
            float ss = 0.f;
#pragma unroll
            for (int m = 0; m < CONV_KEEP; ++m) {
                const int e = lane + 32 * m;
                y[m] = e < width ? conv_at(base + e) : 0.f;
                ss = fmaf(y[m], y[m], ss);
            }
            float r = 1.0f;
            if (qk) r = (1.0f / sqrtf(warp_sum(ss) + unit_eps)) * unit_scale;
#pragma unroll
            for (int m = 0; m < CONV_KEEP; ++m) {
                const int e = lane + 32 * m;
                if (e < width) out[(size_t)t * C + base + e] = qk ? y[m] * r : y[m];
            }
            continue;
        }
        float ss = 0.f;                                                  // wider heads: written, then scaled in place
        for (int e = lane; e < width; e += 32) {
            const float y = conv_at(base + e);
            out[(size_t)t * C + base + e] = y;
            ss = fmaf(y, y, ss);
        }
        if (qk) {
            ss = warp_sum(ss);
            const float r = (1.0f / sqrtf(ss + unit_eps)) * unit_scale;
            __syncwarp();
            for (int e = lane; e < width; e += 32) out[(size_t)t * C + base + e] *= r;
        }
    }
}

// The same for steps of many tokens: a block a (request, chunk of `tt` tokens, head); the chunk's rows of the head, with the
// taps - 1 rows in front of them, and the head's weights are brought into shared memory once (all loads in flight), then a warp
// a token.  The arithmetic of an output is conv_prep_kernel's, operation for operation, so both give the same bits.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) conv_prep_tile_kernel(const TA* __restrict__ proj, int stride, const TW* __restrict__ taps_w, int taps,
                                                             const float* __restrict__ conv_state, long long slot_stride,
                                                             const int* __restrict__ q_start, const int* __restrict__ slots,
                                                             float* __restrict__ out, int C, int nqk, int d, int nv, int dv,
                                                             float unit_eps, float q_scale, int tt) {
    extern __shared__ float sm[];                        // rows [tt + taps - 1][width], then weights [width][taps]
    const int b = blockIdx.x, u = blockIdx.z, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const int c0 = t0 + blockIdx.y * tt, c1 = min(t1, c0 + tt);
    if (c0 >= t1) return;
    const bool qk = u < 2 * nqk;
    const int width = qk ? d : dv, base = qk ? u * d : 2 * nqk * d + (u - 2 * nqk) * dv;
    const float* st = conv_state + (size_t)slots[b] * slot_stride;
    float* ws = sm + (size_t)(tt + taps - 1) * width;
    const int nrows = (c1 - c0) + taps - 1, first = (c0 - t0) - (taps - 1);       // place in the step of the tile's first row
    int shift = 0;                                       // threads a row: the power of two that holds the head (no division an element)
    while ((1 << shift) < width) ++shift;
    const int e = threadIdx.x & ((1 << shift) - 1), rows_a_pass = blockDim.x >> shift;
    if (e < width) {
        for (int r = threadIdx.x >> shift; r < nrows; r += rows_a_pass) {
            const int src = first + r;
            sm[r * width + e] = src >= 0 ? to_f<TA>(proj[(size_t)(t0 + src) * stride + base + e])
                                         : st[(size_t)(taps - 1 + src) * C + base + e];
        }
    }
    for (int i = threadIdx.x; i < width * taps; i += blockDim.x) ws[i] = to_f<TW>(taps_w[(size_t)base * taps + i]);
    __syncthreads();
    const float unit_scale = u < nqk ? q_scale : 1.0f;
    for (int t = c0 + wid; t < c1; t += 8) {
        const float* rows = sm + (size_t)(t - c0) * width;               // the row taps - 1 tokens back
        float y[CONV_KEEP];
        float ss = 0.f;
#pragma unroll
        for (int m = 0; m < CONV_KEEP; ++m) {
            const int el = lane + 32 * m;
            float v = 0.f;
            if (el < width) {
                float acc = 0.f;
                for (int j = 0; j < taps; ++j) acc = fmaf(ws[el * taps + j], rows[(size_t)j * width + el], acc);
                v = acc / (1.0f + expf(-acc));
            }
            y[m] = v;
            ss = fmaf(v, v, ss);
        }
        float r = 1.0f;
        if (qk) r = (1.0f / sqrtf(warp_sum(ss) + unit_eps)) * unit_scale;
#pragma unroll
        for (int m = 0; m < CONV_KEEP; ++m) {
            const int el = lane + 32 * m;
            if (el < width) out[(size_t)t * C + base + el] = qk ? y[m] * r : y[m];
        }
    }
}

// The slot's inputs after the step: the last taps - 1 of (what the slot held, then the step's inputs).  A thread a channel;
// going from the oldest place on, every place reads a place behind it or the step's rows, so nothing is read after it
// was overwritten.
template <typename TA>
__global__ void conv_keep_kernel(const TA* __restrict__ proj, int stride, int taps, float* __restrict__ conv_state, long long slot_stride,
                                 const int* __restrict__ q_start, const int* __restrict__ slots, int C) {
    const int b = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int t0 = q_start[b], n = q_start[b + 1] - t0;
    if (n <= 0) return;
    float* st = conv_state + (size_t)slots[b] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int j = 0; j < taps - 1; ++j) {
            const int src = n - (taps - 1) + j;                          // place in the step; negative: still the slot's
            st[(size_t)j * C + c] = src >= 0 ? to_f<TA>(proj[(size_t)(t0 + src) * stride + c]) : st[(size_t)(j + n) * C + c];
        }
    }
}

TL_EXPORT int tl_conv_prep(const void* proj, int act_dtype, int stride, const void* taps_w, int w_dtype, int taps, float* conv_state,
                           long long slot_stride, const int* q_start, const int* slots, float* out, int B, int max_q_len,
                           int nqk, int d, int nv, int dv, float unit_eps, float q_scale, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    if (taps < 1 || (taps > 1 && !conv_state)) return 1;
    const int C = 2 * nqk * d + nv * dv;
    // steps of many tokens with heads of up to 32 * CONV_KEEP: the tile kernel, as many tokens a block as 40 KB of rows hold
    const int widest = d > dv ? d : dv;
    int tt = (int)(40 * 1024 / sizeof(float)) / widest - (taps - 1);
    tt = tt > 32 ? 32 : tt;
    if (max_q_len >= 16 && widest <= 32 * CONV_KEEP && tt >= 8 && 2 * nqk + nv <= 65535) {
        const dim3 grid(B, (max_q_len + tt - 1) / tt, 2 * nqk + nv);
        if (grid.y > 65535) return 1;
        const size_t smem = ((size_t)(tt + taps - 1) * widest + (size_t)widest * taps) * sizeof(float);
        if (smem > 48 * 1024) return 1;
#define CT(TA, TW) launch_after_wait(conv_prep_tile_kernel<TA, TW>, grid, dim3(256), smem, stream, (const TA*)proj, stride, (const TW*)taps_w, taps, \
        (const float*)conv_state, slot_stride, q_start, slots, out, C, nqk, d, nv, dv, unit_eps, q_scale, tt)
        if (act_dtype == TL_F32) { if (w_dtype == TL_F32) CT(float, float); else CT(float, bf16); }
        else { if (w_dtype == TL_F32) CT(bf16, float); else CT(bf16, bf16); }
#undef CT
    } else {
        const dim3 grid(B, (max_q_len + DELTA_TOK - 1) / DELTA_TOK, (2 * nqk + nv + 3) / 4);
        if (grid.y > 65535 || grid.z > 65535) return 1;
#define CP(TA, TW) launch_after_wait(conv_prep_kernel<TA, TW>, grid, dim3(128), 0, stream, (const TA*)proj, stride, (const TW*)taps_w, taps, \
        (const float*)conv_state, slot_stride, q_start, slots, out, C, nqk, d, nv, dv, unit_eps, q_scale)
        if (act_dtype == TL_F32) { if (w_dtype == TL_F32) CP(float, float); else CP(float, bf16); }
        else { if (w_dtype == TL_F32) CP(bf16, float); else CP(bf16, bf16); }
#undef CP
    }
    int e = tl_launch_status();
    if (e || taps == 1) return e;
    const dim3 kgrid(B, (C + 255) / 256 < 64 ? (C + 255) / 256 : 64);
    if (act_dtype == TL_F32) launch_after_wait(conv_keep_kernel<float>, kgrid, dim3(256), 0, stream, (const float*)proj, stride, taps, conv_state, slot_stride, q_start, slots, C);
    else launch_after_wait(conv_keep_kernel<bf16>, kgrid, dim3(256), 0, stream, (const bf16*)proj, stride, taps, conv_state, slot_stride, q_start, slots, C);
    return tl_launch_status();
}

// ------------------------------------------------------------------ the recurrence
struct DeltaArgs {
    const float* qkv; int stride;          // [T, stride] float: q [nqk, d], k [nqk, d], v [H, dv] as conv_prep left them
    int q_off, k_off, v_off;
    const float* gates; int gate_stride;   // [T, >= 2 H]: b_t (beta's pre-activation) then a_t (the decay's), per head
    const float* A_log; const float* dt_bias;      // [H]
    float* state; long long slot_stride;
    const int* q_start; const int* slots;
    float* out;                            // [T, H * dv]
    int H, nqk, d, dv;
};

template <int R, int IS> struct DeltaShape {
    static constexpr int NT = IS * DELTA_JS;
    static constexpr int PB = R * NT;                            // floats of state a (head, column slice)
    static constexpr int RS = R + 4;                             // padded: the IS threads of a column read different banks
    static constexpr int TS = IS * RS;
    static constexpr int CH = IS >= 32 ? DELTA_C / 2 : DELTA_C;  // tokens a chunk: q and k of a chunk stay under 48 KB
};

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// AHEAD: the next chunk's rows wait in registers while a chunk is worked through (requests of more tokens than a chunk); without
// it the kernel needs 48 registers instead of 120 and more blocks share an SM, which is what a step of single tokens, all
// loads and stores of state, wants.  The arithmetic is the same.
// COMP (the 32-bit engine): every state element is a pair of floats, S + L, where L gathers what the roundings of S lose: the
// decay and the write are done as error-free steps (the exact error of a product by a fused multiply-add, of a sum by the six
// additions of the two-sum), and both column sums read S and L.  A float state gathers one rounding a token, and its read-out
// is a small difference of large sums: after a thousand tokens that is a relative error of 2e-5 in the read-out; the pair
// keeps it near 1e-6, the level of the sums themselves.  The slot holds S, then L.  The decay is a pair as well, g = gh + gl:
// a decay just under one loses up to 3e-8 of itself when it is rounded to a float, the same 3e-8 every time the same token
// comes again, so a far token's weight, a product of a thousand decays, would be off by 3e-5; gl = expm1(x) - (gh - 1) holds
// what gh = exp(x) lost (x, the small exponent, carries it).
template <int R, int IS, bool AHEAD, bool COMP>
__global__ void __launch_bounds__(DeltaShape<R, IS>::NT) delta_scan_kernel(const DeltaArgs A) {
    using Sh = DeltaShape<R, IS>;
    constexpr int NT = Sh::NT, PB = Sh::PB, RS = Sh::RS, TS = Sh::TS, CH = Sh::CH;
    __shared__ __align__(16) float qs[CH * TS];
    __shared__ __align__(16) float ks[CH * TS];
    __shared__ float vs[CH * DELTA_JS];
    __shared__ float gg[CH], gb[CH], gl[COMP ? CH : 1];
    const int d = A.d;
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int hq = h / (A.H / A.nqk);                            // the q/k head this value head reads
    const int tid = threadIdx.x, islice = tid % IS, j = tid / IS;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int t0 = A.q_start[b], t1 = A.q_start[b + 1];
    if (t0 >= t1) return;
    float* st = A.state + (size_t)A.slots[b] * A.slot_stride + ((size_t)h * gridDim.z + z) * (COMP ? 2 * PB : PB);
    float S[R], L[COMP ? R : 1];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = st[r * NT + tid];
    if constexpr (COMP) {
#pragma unroll
        for (int r = 0; r < R; ++r) L[r] = st[PB + r * NT + tid];
    }
    const int jcol = z * DELTA_JS + j;
    const bool live = jcol < A.dv;
    const float neg_rate = -expf(A.A_log[h]), bias = A.dt_bias[h];
    for (int i = tid; i < CH * TS; i += NT) { qs[i] = 0.f; ks[i] = 0.f; }     // rows beyond d stay zero
    // AHEAD: which elements of a chunk this thread moves never changes, so it is worked out once, and the next chunk's q, k, v
    // and gate pre-activations wait in registers while this chunk is worked through.
    constexpr int PF = AHEAD ? CH * R / DELTA_JS : 1;            // q (and k) elements of a chunk a thread fetches (CH R IS / NT)
    constexpr int PV = AHEAD ? (CH * DELTA_JS + NT - 1) / NT : 1;
    int g_off[PF], s_off[PF], tok_of[PF], v_goff[PV];
    unsigned v_ok = 0;
    float fq[PF], fk[PF], fv[PV], fgb = 0.f, fga = 0.f;
    if constexpr (AHEAD) {
#pragma unroll
        for (int it = 0; it < PF; ++it) {
            const int idx = tid + it * NT, t = idx / d, e = idx - t * d;
            tok_of[it] = t < CH ? t : CH;                        // CH: beyond every chunk
            g_off[it] = t * A.stride + hq * d + e;
            s_off[it] = t * TS + (e / R) * RS + (e % R);
        }
#pragma unroll
        for (int it = 0; it < PV; ++it) {
            const int idx = tid + it * NT, t = idx / DELTA_JS, col = z * DELTA_JS + (idx - t * DELTA_JS);
            v_goff[it] = t * A.stride + A.v_off + h * A.dv + col;
            if (t < CH && col < A.dv) v_ok |= 1u << it;
        }
    }
    auto fetch = [&](int c0) {
        const int n = min(CH, t1 - c0);
        const float* base = A.qkv + (size_t)c0 * A.stride;
#pragma unroll
        for (int it = 0; it < PF; ++it)
            if (tok_of[it] < n) { fq[it] = base[g_off[it] + A.q_off]; fk[it] = base[g_off[it] + A.k_off]; }
#pragma unroll
        for (int it = 0; it < PV; ++it)
            if (((v_ok >> it) & 1u) && (tid + it * NT) / DELTA_JS < n) fv[it] = base[v_goff[it]];
        if (tid < n) {
            const float* g = A.gates + (size_t)(c0 + tid) * A.gate_stride;
            fgb = g[h]; fga = g[A.H + h];
        }
    };
    if constexpr (AHEAD) fetch(t0);
    __syncthreads();
    for (int c0 = t0; c0 < t1; c0 += CH) {
        const int n = min(CH, t1 - c0);
        if constexpr (AHEAD) {
#pragma unroll
            for (int it = 0; it < PF; ++it)
                if (tok_of[it] < n) { qs[s_off[it]] = fq[it]; ks[s_off[it]] = fk[it]; }
#pragma unroll
            for (int it = 0; it < PV; ++it) {
                const int idx = tid + it * NT;
                if (idx < n * DELTA_JS) vs[idx] = ((v_ok >> it) & 1u) ? fv[it] : 0.f;
            }
        } else {
            for (int i = tid; i < n * d; i += NT) {
                const int t = i / d, e = i - t * d;
                const float* row = A.qkv + (size_t)(c0 + t) * A.stride + hq * d + e;
                qs[t * TS + (e / R) * RS + (e % R)] = row[A.q_off];
                ks[t * TS + (e / R) * RS + (e % R)] = row[A.k_off];
            }
            for (int i = tid; i < n * DELTA_JS; i += NT) {
                const int t = i / DELTA_JS, col = z * DELTA_JS + (i - t * DELTA_JS);
                vs[i] = col < A.dv ? A.qkv[(size_t)(c0 + t) * A.stride + A.v_off + h * A.dv + col] : 0.f;
            }
            if (tid < n) {
                const float* g = A.gates + (size_t)(c0 + tid) * A.gate_stride;
                fgb = g[h]; fga = g[A.H + h];
            }
        }
        if (tid < n) {
            gb[tid] = 1.0f / (1.0f + expf(-fgb));
            const float x = neg_rate * softplus_f(fga + bias);
            gg[tid] = expf(x);
            if constexpr (COMP) gl[tid] = __fsub_rn(expm1f(x), __fsub_rn(gg[tid], 1.0f));
        }
        __syncthreads();
        if (AHEAD && c0 + CH < t1) fetch(c0 + CH);
        const float* kt = ks + islice * RS;
        const float* qt = qs + islice * RS;
        for (int t = 0; t < n; ++t) {
            // S^T k is taken of the state before the decay and multiplied by g once (the same sum); the decay and the
            // write are then one fused multiply-add an element, so a step rounds the state once, not twice
            const float g = gg[t];
            if constexpr (COMP) {
                float acc = 0.f, accl = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) { acc = fmaf(S[r], kt[t * TS + r], acc); accl = fmaf(L[r], kt[t * TS + r], accl); }
                acc += accl;
#pragma unroll
                for (int o = 1; o < IS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                const float glo = gl[t];
                const float u = gb[t] * (vs[t * DELTA_JS + j] - fmaf(glo, acc, g * acc));
                float rd = 0.f, rdl = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float k = kt[t * TS + r], q = qt[t * TS + r];
                    const float p = __fmul_rn(k, u), pe = __fmaf_rn(k, u, -p);           // k u = p + pe exactly
                    const float gs = __fmul_rn(g, S[r]), gse = __fmaf_rn(g, S[r], -gs);   // g S = gs + gse exactly
                    const float sum = __fadd_rn(gs, p), bb = __fsub_rn(sum, gs);          // gs + p = sum + se exactly
                    const float se = __fadd_rn(__fsub_rn(gs, __fsub_rn(sum, bb)), __fsub_rn(p, bb));
                    L[r] = __fmaf_rn(glo, S[r], __fmaf_rn(g, L[r], __fadd_rn(__fadd_rn(se, gse), pe)));
                    S[r] = sum;
                    rd = fmaf(S[r], q, rd); rdl = fmaf(L[r], q, rdl);
                }
                rd += rdl;
#pragma unroll
                for (int o = 1; o < IS; o <<= 1) rd += __shfl_xor_sync(0xffffffffu, rd, o);
                if (live && islice == 0) A.out[(size_t)(c0 + t) * A.H * A.dv + (size_t)h * A.dv + jcol] = rd;
                continue;
            }
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(kt + t * TS + r);
                acc = fmaf(S[r], kk.x, acc);
                acc = fmaf(S[r + 1], kk.y, acc);
                acc = fmaf(S[r + 2], kk.z, acc);
                acc = fmaf(S[r + 3], kk.w, acc);
            }
#pragma unroll
            for (int o = 1; o < IS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float u = gb[t] * (vs[t * DELTA_JS + j] - g * acc);
            float rd = 0.f;
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(kt + t * TS + r);
                const float4 qq = *reinterpret_cast<const float4*>(qt + t * TS + r);
                S[r] = fmaf(g, S[r], kk.x * u);         rd = fmaf(S[r], qq.x, rd);
                S[r + 1] = fmaf(g, S[r + 1], kk.y * u); rd = fmaf(S[r + 1], qq.y, rd);
                S[r + 2] = fmaf(g, S[r + 2], kk.z * u); rd = fmaf(S[r + 2], qq.z, rd);
                S[r + 3] = fmaf(g, S[r + 3], kk.w * u); rd = fmaf(S[r + 3], qq.w, rd);
            }
#pragma unroll
            for (int o = 1; o < IS; o <<= 1) rd += __shfl_xor_sync(0xffffffffu, rd, o);
            if (live && islice == 0) A.out[(size_t)(c0 + t) * A.H * A.dv + (size_t)h * A.dv + jcol] = rd;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) st[r * NT + tid] = S[r];
    if constexpr (COMP) {
#pragma unroll
        for (int r = 0; r < R; ++r) st[PB + r * NT + tid] = L[r];
    }
}

// How a head of d rows is dealt out: 0: R 4 x IS 8 (d <= 32), 1: 8 x 8 (<= 64), 2: 8 x 16 (<= 128), 3: 8 x 32 (<= 256); -1: too large.
static int delta_shape(int d) { return d <= 32 ? 0 : d <= 64 ? 1 : d <= 128 ? 2 : d <= 256 ? 3 : -1; }

// Floats of state per (head, column slice) for a head of d rows (twice as many with the pair of floats an element); 0: too large.
TL_EXPORT int tl_delta_state_floats(int d, int compensated) {
    const int f = compensated ? 2 : 1;
    switch (delta_shape(d)) {
        case 0: return f * DeltaShape<4, 8>::PB;
        case 1: return f * DeltaShape<8, 8>::PB;
        case 2: return f * DeltaShape<8, 16>::PB;
        case 3: return f * DeltaShape<8, 32>::PB;
    }
    return 0;
}
TL_EXPORT int tl_delta_columns() { return DELTA_JS; }

TL_EXPORT int tl_delta_scan(const float* qkv, int stride, int q_off, int k_off, int v_off, const float* gates, int gate_stride,
                            const float* A_log, const float* dt_bias, float* state, long long slot_stride, const int* q_start,
                            const int* slots, float* out, int B, int H, int nqk, int d, int dv, int max_q_len, int compensated,
                            cudaStream_t stream) {
    if (B <= 0 || H <= 0) return 0;
    if (H > 65535 || nqk < 1 || H % nqk) return 1;
    const DeltaArgs A{qkv, stride, q_off, k_off, v_off, gates, gate_stride, A_log, dt_bias, state, slot_stride, q_start, slots, out,
                      H, nqk, d, dv};
    const dim3 grid(B, H, (dv + DELTA_JS - 1) / DELTA_JS);
#define DSK(R_, IS_, AH, CO) launch_after_wait(delta_scan_kernel<R_, IS_, AH, CO>, grid, dim3(DeltaShape<R_, IS_>::NT), 0, stream, A)
#define DS(R_, IS_) (compensated ? (max_q_len > DeltaShape<R_, IS_>::CH ? DSK(R_, IS_, true, true) : DSK(R_, IS_, false, true)) \
                                 : (max_q_len > DeltaShape<R_, IS_>::CH ? DSK(R_, IS_, true, false) : DSK(R_, IS_, false, false)))
    switch (delta_shape(d)) {
        case 0: return DS(4, 8);
        case 1: return DS(8, 8);
        case 2: return DS(8, 16);
        case 3: return DS(8, 32);
    }
#undef DS
#undef DSK
    return 1;
}
