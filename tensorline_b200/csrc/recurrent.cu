// Linear recurrences with a matrix state per head, and the element-wise steps around them.
//
//   S_t = a_t S_{t-1} + b_t k_t v_t^T        S: [d, dv] per (request, head), float, kept in the request's state slot
//   o_t = S_t^T q_t
//
// Two kinds of (a_t, b_t), one kernel:
//   fixed decay    a_t = decay[h], b_t = 1                                   (retention: no normaliser)
//   gated          log gates i_t = cap tanh(x_i / cap), f_t = logsigmoid(cap tanh(x_f / cap)) from the
//                  pre-activations x_i, x_f; running maximum m_t = max(f_t + m_{t-1}, i_t), m_0 = 0;
//                  a_t = exp(f_t + m_{t-1} - m_t), b_t = exp(i_t - m_t); a normaliser n_t = a_t n_{t-1} + b_t k_t
//                  rides along as one more column of S (v = 1), and
//                  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)   (the matrix memory of the xLSTM)
// q and k may be rotated by position first (either pairing of dimensions, the first `rot` of a head) and scaled.
// Everything is float: angles, gates, exponentials, the state and the sums; only q, k, v come in the
// activation type, as the projection left them.
//
// Work split.  grid (requests, heads, value-column slices of SCAN_JS): a block walks its request's tokens of the
// step in order, SCAN_C at a time.  A thread owns one value column and every SCAN_IS-th row of S in registers
// (R rows), so a token costs it R updates and R products and no synchronisation; the column sums are finished by
// shuffles over the SCAN_IS lanes that share a column.  The sequence of operations on a state element and on an
// output is the same wherever the step was cut, so portions, single tokens and whole prompts give the same bits.
// The state lies in memory as the threads hold it ([row group][thread]; loads and stores of a step of single
// tokens, which are all that step moves, are contiguous); the gated kind keeps m, and each column slice its own
// copy of n and m, behind it.  Nobody else reads the state.
#include "common.cuh"

constexpr int SCAN_IS = 8;
constexpr int SCAN_JS = 16;
constexpr int SCAN_C = 16;

struct ScanArgs {
    const void* proj; int stride;          // the step's projection rows [T, stride]
    int q_off, k_off, v_off;               // where q [H, d], k [H, d], v [H, dv] start inside a row
    const float* gates;                    // gated: [T, 2 H] pre-activations, input gates then forget gates
    float cap;
    const float* decay;                    // fixed decay: [H]
    const float* inv_freq; int rot; int interleaved;
    const int* pos;
    float q_scale, k_scale;
    float* state; long long slot_stride;   // floats per slot
    const int* q_start; const int* slots;
    float* out;                            // [T, H * dv]
    int H, d, dv;
    float den_eps;
};

template <bool GATED> struct ScanShape {
    static constexpr int JW = SCAN_JS + (GATED ? 1 : 0);
    static constexpr int NT = (SCAN_IS * JW + 31) / 32 * 32;
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename TA, int R, bool GATED>
__global__ void __launch_bounds__(ScanShape<GATED>::NT) linear_scan_kernel(const ScanArgs A) {
    constexpr int JW = ScanShape<GATED>::JW, NT = ScanShape<GATED>::NT;
    constexpr int PB = R * NT + (GATED ? 4 : 0);
    extern __shared__ float sm[];
    const int d = A.d;
    float* qs = sm;
    float* ks = qs + SCAN_C * d;
    float* vs = ks + SCAN_C * d;
    float* ga = vs + SCAN_C * SCAN_JS;
    float* gb = ga + SCAN_C;
    float* gm = gb + SCAN_C;
    float* nq = gm + SCAN_C;
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, islice = tid % SCAN_IS, j = tid / SCAN_IS;
    const int t0 = A.q_start[b], t1 = A.q_start[b + 1];
    float* st = A.state + (size_t)A.slots[b] * A.slot_stride + ((size_t)h * gridDim.z + z) * PB;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = st[r * NT + tid];
    float m_run = GATED ? st[R * NT] : 0.f;
    const int jcol = z * SCAN_JS + j;
    const bool ones = GATED && j == SCAN_JS;
    const bool live = j < SCAN_JS && jcol < A.dv;
    const float dec = GATED ? 0.f : A.decay[h];
    const TA* proj = (const TA*)A.proj;
    const int rhalf = A.rot >> 1;

    for (int c0 = t0; c0 < t1; c0 += SCAN_C) {
        const int n = min(SCAN_C, t1 - c0);
        // q and k of the chunk: rotation by position, then the scale
        for (int idx = tid; idx < n * d; idx += NT) {
            const int t = idx / d, e = idx - t * d;
            const TA* row = proj + (size_t)(c0 + t) * A.stride + (size_t)h * d;
            float qv = to_f<TA>(row[A.q_off + e]), kv = to_f<TA>(row[A.k_off + e]);
            if (e < A.rot) {
                int i, partner; float sign;
                if (A.interleaved) { i = e >> 1; partner = e ^ 1; sign = (e & 1) ? 1.f : -1.f; }
                else { i = e < rhalf ? e : e - rhalf; partner = e < rhalf ? e + rhalf : e - rhalf; sign = e < rhalf ? -1.f : 1.f; }
                float s, c;
                sincosf(__fmul_rn((float)A.pos[c0 + t], A.inv_freq[i]), &s, &c);
                const float qp = to_f<TA>(row[A.q_off + partner]), kp = to_f<TA>(row[A.k_off + partner]);
                qv = __fmul_rn(qv, c) + sign * __fmul_rn(qp, s);
                kv = __fmul_rn(kv, c) + sign * __fmul_rn(kp, s);
            }
            qs[t * d + e] = qv * A.q_scale;
            ks[t * d + e] = kv * A.k_scale;
        }
        for (int idx = tid; idx < n * SCAN_JS; idx += NT) {
            const int t = idx / SCAN_JS, jj = idx - t * SCAN_JS, col = z * SCAN_JS + jj;
            vs[idx] = col < A.dv ? to_f<TA>(proj[(size_t)(c0 + t) * A.stride + A.v_off + (size_t)h * A.dv + col]) : 0.f;
        }
        if (GATED) {
            if (tid < n) {
                const float* g = A.gates + (size_t)(c0 + tid) * 2 * A.H;
                gb[tid] = A.cap * tanhf(g[h] / A.cap);
                ga[tid] = log_sigmoid(A.cap * tanhf(g[A.H + h] / A.cap));
            }
            __syncthreads();
            if (tid == 0) {                              // the running maximum is the only serial part
                float m = m_run;
                for (int t = 0; t < n; ++t) { m = fmaxf(ga[t] + m, gb[t]); gm[t] = m; }
            }
            __syncthreads();
            float a = 0.f, bb = 0.f;
            if (tid < n) {
                const float mp = tid ? gm[tid - 1] : m_run, mn = gm[tid];
                a = expf(ga[tid] + mp - mn);
                bb = expf(gb[tid] - mn);
            }
            __syncthreads();                             // every thread has read the log gates it needs
            if (tid < n) { ga[tid] = a; gb[tid] = bb; }
        }
        __syncthreads();
        if (GATED) m_run = gm[n - 1];

        float po[SCAN_C];
#pragma unroll
        for (int t = 0; t < SCAN_C; ++t) {
            po[t] = 0.f;
            if (t < n) {
                const float a = GATED ? ga[t] : dec;
                const float v = ones ? 1.f : (live ? vs[t * SCAN_JS + j] : 0.f);
                const float bv = GATED ? gb[t] * v : v;
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = r * SCAN_IS + islice;
                    if (i < d) {
                        S[r] = fmaf(a, S[r], ks[t * d + i] * bv);
                        acc = fmaf(S[r], qs[t * d + i], acc);
                    }
                }
                po[t] = acc;
            }
        }
#pragma unroll
        for (int t = 0; t < SCAN_C; ++t) {
            po[t] += __shfl_xor_sync(0xffffffffu, po[t], 1);
            po[t] += __shfl_xor_sync(0xffffffffu, po[t], 2);
            po[t] += __shfl_xor_sync(0xffffffffu, po[t], 4);
        }
        if (GATED) {
            if (ones && islice == 0) {
#pragma unroll
                for (int t = 0; t < SCAN_C; ++t) if (t < n) nq[t] = po[t];
            }
            __syncthreads();
        }
        if (live && islice == 0) {
#pragma unroll
            for (int t = 0; t < SCAN_C; ++t) {
                if (t < n) {
                    float o = po[t];
                    if (GATED) o = o / (fmaxf(fabsf(nq[t]), expf(-gm[t])) + A.den_eps);
                    A.out[(size_t)(c0 + t) * A.H * A.dv + (size_t)h * A.dv + jcol] = o;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) st[r * NT + tid] = S[r];
    if (GATED && tid == 0) st[R * NT] = m_run;
}

// Floats of state per (head, column slice) for a head of d rows; 0: d is too large.
static int scan_rows(int d) { return d <= 32 ? 4 : d <= 64 ? 8 : d <= 128 ? 16 : d <= 256 ? 32 : 0; }

TL_EXPORT int tl_scan_state_floats(int d, int gated) {
    const int R = scan_rows(d);
    if (!R) return 0;
    return gated ? R * ScanShape<true>::NT + 4 : R * ScanShape<false>::NT;
}
TL_EXPORT int tl_scan_columns() { return SCAN_JS; }

template <typename TA, bool GATED>
static int launch_scan(const ScanArgs& A, int B, cudaStream_t stream) {
    const int nz = (A.dv + SCAN_JS - 1) / SCAN_JS;
    const dim3 grid(B, A.H, nz), block(ScanShape<GATED>::NT);
    const size_t smem = (size_t)(2 * SCAN_C * A.d + SCAN_C * SCAN_JS + 4 * SCAN_C) * sizeof(float);
    switch (scan_rows(A.d)) {
        case 4: linear_scan_kernel<TA, 4, GATED><<<grid, block, smem, stream>>>(A); break;
        case 8: linear_scan_kernel<TA, 8, GATED><<<grid, block, smem, stream>>>(A); break;
        case 16: linear_scan_kernel<TA, 16, GATED><<<grid, block, smem, stream>>>(A); break;
        case 32: linear_scan_kernel<TA, 32, GATED><<<grid, block, smem, stream>>>(A); break;
        default: return 1;
    }
    return tl_launch_status();
}

TL_EXPORT int tl_linear_scan(const void* proj, int act_dtype, int stride, int q_off, int k_off, int v_off,
                             const float* gates, float cap, const float* decay, const float* inv_freq, int rot,
                             int interleaved, const int* pos, float q_scale, float k_scale, float* state,
                             long long slot_stride, const int* q_start, const int* slots, float* out, int B, int H,
                             int d, int dv, float den_eps, cudaStream_t stream) {
    if (B <= 0 || H <= 0) return 0;
    if (B > 65535 * 32768 || H > 65535 || (rot & 1) || rot > d) return 1;
    const ScanArgs A{proj, stride, q_off, k_off, v_off, gates, cap, decay, inv_freq, rot, interleaved, pos, q_scale, k_scale,
                     state, slot_stride, q_start, slots, out, H, d, dv, den_eps};
    const bool gated = gates != nullptr;
    if (act_dtype == TL_F32) return gated ? launch_scan<float, true>(A, B, stream) : launch_scan<float, false>(A, B, stream);
    return gated ? launch_scan<bf16, true>(A, B, stream) : launch_scan<bf16, false>(A, B, stream);
}

// ------------------------------------------------------------------ per-head RMS norm, weight, gate
// out[t, h, j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * (w ? w[h dv + j] : 1) * act(g[t, h dv + j]); one warp per
// (token, head); act 0: no gate, 1: sigmoid, 2: silu.  o is float, g and out of the activation type.
template <typename TA, typename TW>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const TA* __restrict__ g, int g_stride,
                                      const TW* __restrict__ w, TA* __restrict__ out, int H, int dv, float eps, int act) {
    const int t = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= H) return;
    const float* row = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int j = lane; j < dv; j += 32) {
        float v = row[j] * rstd;
        if (w) v *= to_f<TW>(w[h * dv + j]);
        if (act) {
            const float x = to_f<TA>(g[(size_t)t * g_stride + h * dv + j]);
            const float s = 1.0f / (1.0f + expf(-x));
            v *= act == 1 ? s : x * s;
        }
        out[((size_t)t * H + h) * dv + j] = from_f<TA>(v);
    }
}

TL_EXPORT int tl_head_norm_gate(const float* o, const void* g, int g_stride, const void* w, int w_dtype, void* out,
                                int act_dtype, int T, int H, int dv, float eps, int act, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    const dim3 grid(T, (H + 3) / 4), block(128);
#define HNG(TA, TW) head_norm_gate_kernel<TA, TW><<<grid, block, 0, stream>>>(o, (const TA*)g, g_stride, (const TW*)w, (TA*)out, H, dv, eps, act)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) HNG(float, float); else HNG(float, bf16); }
    else { if (w_dtype == TL_F32) HNG(bf16, float); else HNG(bf16, bf16); }
#undef HNG
    return tl_launch_status();
}

// ------------------------------------------------------------------ mean of two normalised branches
// out = c * (a / rms(a) * wa + b / rms(b) * wb) over the model width, one block per token, statistics in float.
template <typename TA, typename TW>
__global__ void sum_normed_kernel(const TA* __restrict__ a, const TA* __restrict__ b, const TW* __restrict__ wa,
                                  const TW* __restrict__ wb, TA* __restrict__ out, int W, float eps, float c) {
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * W;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float x = to_f<TA>(a[base + i]), y = to_f<TA>(b[base + i]);
        sa = fmaf(x, x, sa); sb = fmaf(y, y, sb);
    }
    sa = block_sum(sa, red);
    sb = block_sum(sb, red);
    const float ra = 1.0f / sqrtf(sa / (float)W + eps), rb = 1.0f / sqrtf(sb / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float x = to_f<TA>(a[base + i]) * ra * to_f<TW>(wa[i]), y = to_f<TA>(b[base + i]) * rb * to_f<TW>(wb[i]);
        out[base + i] = from_f<TA>(c * (x + y));
    }
}

TL_EXPORT int tl_sum_normed(const void* a, const void* b, const void* wa, const void* wb, int w_dtype, void* out,
                            int act_dtype, int T, int W, float eps, float c, cudaStream_t stream) {
    if (T <= 0) return 0;
#define SN(TA, TW) sum_normed_kernel<TA, TW><<<T, 256, 0, stream>>>((const TA*)a, (const TA*)b, (const TW*)wa, (const TW*)wb, (TA*)out, W, eps, c)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) SN(float, float); else SN(float, bf16); }
    else { if (w_dtype == TL_F32) SN(bf16, float); else SN(bf16, bf16); }
#undef SN
    return tl_launch_status();
}
