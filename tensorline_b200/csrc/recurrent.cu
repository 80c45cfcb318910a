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
// step in order, SCAN_C at a time.  A thread owns one value column and R consecutive rows of S in registers (IS
// threads a column, R * IS >= d), so a token costs it R updates and R products and no synchronisation; the column
// sums are finished by shuffles over the IS lanes that share a column.  The sequence of operations on a state element and on an
// output is the same wherever the step was cut, so portions, single tokens and whole prompts give the same bits.
// The state lies in memory as the threads hold it ([row group][thread]; loads and stores of a step of single
// tokens, which are all that step moves, are contiguous); the gated kind keeps m, and each column slice its own
// copy of n and m, behind it.  Nobody else reads the state.
#include "common.cuh"

constexpr int SCAN_JS = 16;      // value columns a block
constexpr int SCAN_C = 16;       // tokens a chunk

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

// A head's d rows are dealt out to IS threads a column, R consecutive rows each (R * IS >= d; the rows beyond d are zeros).
template <int R, int IS, bool GATED> struct ScanShape {
    static constexpr int JW = SCAN_JS + (GATED ? 1 : 0);
    static constexpr int NT = (IS * JW + 31) / 32 * 32;
    static constexpr int PB = R * NT + (GATED ? 4 : 0);          // floats of state a (head, column slice)
    static constexpr int RS = R + 4;                             // a thread's rows of q or k in shared memory, padded: the
    static constexpr int TS = IS * RS;                           // 16-byte reads of the IS threads of a column hit different banks
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename TA, int R, int IS, bool GATED>
__global__ void __launch_bounds__(ScanShape<R, IS, GATED>::NT) linear_scan_kernel(const ScanArgs A) {
    using Sh = ScanShape<R, IS, GATED>;
    constexpr int NT = Sh::NT, PB = Sh::PB, RS = Sh::RS, TS = Sh::TS;
    constexpr int PF = (SCAN_C * R * IS + NT - 1) / NT;           // q (and k) elements of a chunk a thread fetches
    constexpr int PV = (SCAN_C * SCAN_JS + NT - 1) / NT;          // v elements
    extern __shared__ __align__(16) float sm[];
    const int d = A.d;
    float* qs = sm;                                                // [C][IS][RS]
    float* ks = qs + SCAN_C * TS;
    float* vs = ks + SCAN_C * TS;                                  // [C][JS]
    float* ga = vs + SCAN_C * SCAN_JS;
    float* gb = ga + SCAN_C;
    float* gm = gb + SCAN_C;
    float* nq = gm + SCAN_C;
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, islice = tid % IS, j = tid / IS;
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
    // rows beyond d and the padding stay zero; a step of single tokens uses (and clears) the first token's part only
    const int used = min(SCAN_C, t1 - t0) * TS;
    for (int i = tid; i < used; i += NT) { qs[i] = 0.f; ks[i] = 0.f; }

    // Which elements of a chunk this thread moves never changes: token and dimension of each, its place in the chunk's rows
    // of the projection and in shared memory, worked out once.
    int g_off[PF], s_off[PF], v_goff[PV];
    unsigned in_rot = 0, v_ok = 0;                         // bit it: the element is rotated / the v element exists
    int tok_of[PF];
#pragma unroll
    for (int it = 0; it < PF; ++it) {
        const int idx = tid + it * NT, t = idx / d, e = idx - t * d;
        tok_of[it] = t < SCAN_C ? t : SCAN_C;              // SCAN_C: beyond every chunk
        g_off[it] = t * A.stride + h * d + e;
        s_off[it] = t * TS + (e / R) * RS + (e % R);
        if (e < A.rot) in_rot |= 1u << it;
    }
#pragma unroll
    for (int it = 0; it < PV; ++it) {
        const int idx = tid + it * NT, t = idx / SCAN_JS, col = z * SCAN_JS + (idx - t * SCAN_JS);
        v_goff[it] = t * A.stride + A.v_off + h * A.dv + col;
        if (t < SCAN_C && col < A.dv) v_ok |= 1u << it;
    }
    float* freq = nq + SCAN_C;                             // [rot / 2]
    for (int i = tid; i < rhalf; i += NT) freq[i] = A.inv_freq[i];
    const int pos0 = t0 < t1 ? A.pos[t0] : 0;              // a request's tokens of a step are consecutive positions

    // The next chunk's q, k, v (as the projection left them) and gate pre-activations wait in registers, unconverted, while
    // this chunk is worked through: their loads are issued before the chunk's arithmetic and first used after it.
    TA fq[PF], fk[PF], fv[PV];
    float fgi = 0.f, fgf = 0.f;
    auto fetch = [&](int c0) {
        const int n = min(SCAN_C, t1 - c0);
        const TA* base = proj + (size_t)c0 * A.stride;
#pragma unroll
        for (int it = 0; it < PF; ++it) {
            if (tok_of[it] < n) { fq[it] = base[g_off[it] + A.q_off]; fk[it] = base[g_off[it] + A.k_off]; }
        }
#pragma unroll
        for (int it = 0; it < PV; ++it)
            if (((v_ok >> it) & 1u) && (tid + it * NT) / SCAN_JS < n) fv[it] = base[v_goff[it]];
        if (GATED && tid < n) {
            const float* g = A.gates + (size_t)(c0 + tid) * 2 * A.H;
            fgi = g[h]; fgf = g[A.H + h];
        }
    };
    // element e of token t of the chunk in qs / ks
    auto at = [&](int t, int e) { return t * TS + (e / R) * RS + (e % R); };
    if (t0 < t1) fetch(t0);
    __syncthreads();

    for (int c0 = t0; c0 < t1; c0 += SCAN_C) {
        const int n = min(SCAN_C, t1 - c0);
        // the chunk into shared memory; dimensions that are not rotated get their scale here
#pragma unroll
        for (int it = 0; it < PF; ++it) {
            if (tok_of[it] < n) {
                const bool rt = (in_rot >> it) & 1u;
                qs[s_off[it]] = rt ? to_f<TA>(fq[it]) : to_f<TA>(fq[it]) * A.q_scale;
                ks[s_off[it]] = rt ? to_f<TA>(fk[it]) : to_f<TA>(fk[it]) * A.k_scale;
            }
        }
#pragma unroll
        for (int it = 0; it < PV; ++it) {
            const int idx = tid + it * NT;
            if (idx < n * SCAN_JS) vs[idx] = ((v_ok >> it) & 1u) ? to_f<TA>(fv[it]) : 0.f;
        }
        if (GATED && tid < n) {
            gb[tid] = A.cap * tanhf(fgi / A.cap);
            ga[tid] = log_sigmoid(A.cap * tanhf(fgf / A.cap));
        }
        __syncthreads();
        // rotation by position, a pair of dimensions a thread, then the scale
        for (int p = tid; p < n * rhalf; p += NT) {
            const int t = p / rhalf, i = p - t * rhalf;
            const int e1 = at(t, A.interleaved ? 2 * i : i), e2 = at(t, A.interleaved ? 2 * i + 1 : i + rhalf);
            float sn, cs;
            sincosf(__fmul_rn((float)(pos0 + (c0 - t0) + t), freq[i]), &sn, &cs);
            const float q1 = qs[e1], q2 = qs[e2], k1 = ks[e1], k2 = ks[e2];
            qs[e1] = (__fmul_rn(q1, cs) - __fmul_rn(q2, sn)) * A.q_scale;
            qs[e2] = (__fmul_rn(q2, cs) + __fmul_rn(q1, sn)) * A.q_scale;
            ks[e1] = (__fmul_rn(k1, cs) - __fmul_rn(k2, sn)) * A.k_scale;
            ks[e2] = (__fmul_rn(k2, cs) + __fmul_rn(k1, sn)) * A.k_scale;
        }
        if (GATED) {
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
        if (c0 + SCAN_C < t1) fetch(c0 + SCAN_C);

        float po[SCAN_C];
        const float* kt = ks + islice * RS;
        const float* qt = qs + islice * RS;
#pragma unroll
        for (int t = 0; t < SCAN_C; ++t) {
            po[t] = 0.f;
            if (t < n) {
                const float a = GATED ? ga[t] : dec;
                const float v = ones ? 1.f : (live ? vs[t * SCAN_JS + j] : 0.f);
                const float bv = GATED ? gb[t] * v : v;
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const float4 kk = *reinterpret_cast<const float4*>(kt + t * TS + r);
                    const float4 qq = *reinterpret_cast<const float4*>(qt + t * TS + r);
                    S[r] = fmaf(a, S[r], kk.x * bv);         acc = fmaf(S[r], qq.x, acc);
                    S[r + 1] = fmaf(a, S[r + 1], kk.y * bv); acc = fmaf(S[r + 1], qq.y, acc);
                    S[r + 2] = fmaf(a, S[r + 2], kk.z * bv); acc = fmaf(S[r + 2], qq.z, acc);
                    S[r + 3] = fmaf(a, S[r + 3], kk.w * bv); acc = fmaf(S[r + 3], qq.w, acc);
                }
                po[t] = acc;
            }
        }
#pragma unroll
        for (int t = 0; t < SCAN_C; ++t) {
#pragma unroll
            for (int o = 1; o < IS; o <<= 1) po[t] += __shfl_xor_sync(0xffffffffu, po[t], o);
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

// The same recurrence for a step of single tokens (decoding): one token a request, so none of the chunk machinery; a
// block loads its part of the state, brings the token's q and k into shared memory (rotated and scaled by the scan
// kernel's own arithmetic, so a token decoded alone gets the bits it gets inside a portion), works the token in and
// stores the state.  Few registers: several blocks share an SM and the loads and stores of the state, which are all
// the step moves, overlap.
template <typename TA, int R, int IS, bool GATED>
__global__ void __launch_bounds__(ScanShape<R, IS, GATED>::NT) linear_step_kernel(const ScanArgs A) {
    using Sh = ScanShape<R, IS, GATED>;
    constexpr int NT = Sh::NT, PB = Sh::PB, RS = Sh::RS, TS = Sh::TS;
    __shared__ __align__(16) float qs[TS];
    __shared__ __align__(16) float ks[TS];
    __shared__ float sc[4];                                // a, b, m after the token, n . q
    const int d = A.d;
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, islice = tid % IS, j = tid / IS;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
    const int t = A.q_start[b];
    float* st = A.state + (size_t)A.slots[b] * A.slot_stride + ((size_t)h * gridDim.z + z) * PB;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = st[r * NT + tid];
    const float m_run = GATED ? st[R * NT] : 0.f;
    const int jcol = z * SCAN_JS + j;
    const bool ones = GATED && j == SCAN_JS;
    const bool live = j < SCAN_JS && jcol < A.dv;
    const TA* row = (const TA*)A.proj + (size_t)t * A.stride;
    const int rhalf = A.rot >> 1;
    const float vraw = live ? to_f<TA>(row[A.v_off + (size_t)h * A.dv + jcol]) : 0.f;
    for (int e = tid; e < R * IS; e += NT) {
        float qv = 0.f, kv = 0.f;
        if (e < d) {
            qv = to_f<TA>(row[A.q_off + (size_t)h * d + e]); kv = to_f<TA>(row[A.k_off + (size_t)h * d + e]);
            if (e >= A.rot) { qv *= A.q_scale; kv *= A.k_scale; }
        }
        qs[(e / R) * RS + (e % R)] = qv; ks[(e / R) * RS + (e % R)] = kv;
    }
    if (GATED && tid == 0) {
        const float* g = A.gates + (size_t)t * 2 * A.H;
        const float gi = A.cap * tanhf(g[h] / A.cap);
        const float gf = log_sigmoid(A.cap * tanhf(g[A.H + h] / A.cap));
        const float m = fmaxf(gf + m_run, gi);
        sc[0] = expf(gf + m_run - m); sc[1] = expf(gi - m); sc[2] = m;
    }
    __syncthreads();
    if (rhalf) {
        const int p0 = A.pos[t];
        for (int i = tid; i < rhalf; i += NT) {
            const int a1 = A.interleaved ? 2 * i : i, a2 = A.interleaved ? 2 * i + 1 : i + rhalf;
            const int e1 = (a1 / R) * RS + (a1 % R), e2 = (a2 / R) * RS + (a2 % R);
            float sn, cs;
            sincosf(__fmul_rn((float)p0, A.inv_freq[i]), &sn, &cs);
            const float q1 = qs[e1], q2 = qs[e2], k1 = ks[e1], k2 = ks[e2];
            qs[e1] = (__fmul_rn(q1, cs) - __fmul_rn(q2, sn)) * A.q_scale;
            qs[e2] = (__fmul_rn(q2, cs) + __fmul_rn(q1, sn)) * A.q_scale;
            ks[e1] = (__fmul_rn(k1, cs) - __fmul_rn(k2, sn)) * A.k_scale;
            ks[e2] = (__fmul_rn(k2, cs) + __fmul_rn(k1, sn)) * A.k_scale;
        }
        __syncthreads();
    }
    const float a = GATED ? sc[0] : A.decay[h];
    const float v = ones ? 1.f : vraw;
    const float bv = GATED ? sc[1] * v : v;
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < R; r += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(ks + islice * RS + r);
        const float4 qq = *reinterpret_cast<const float4*>(qs + islice * RS + r);
        S[r] = fmaf(a, S[r], kk.x * bv);         acc = fmaf(S[r], qq.x, acc);
        S[r + 1] = fmaf(a, S[r + 1], kk.y * bv); acc = fmaf(S[r + 1], qq.y, acc);
        S[r + 2] = fmaf(a, S[r + 2], kk.z * bv); acc = fmaf(S[r + 2], qq.z, acc);
        S[r + 3] = fmaf(a, S[r + 3], kk.w * bv); acc = fmaf(S[r + 3], qq.w, acc);
    }
#pragma unroll
    for (int o = 1; o < IS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
#pragma unroll
    for (int r = 0; r < R; ++r) st[r * NT + tid] = S[r];
    if (GATED) {
        if (ones && islice == 0) sc[3] = acc;
        if (tid == 0) st[R * NT] = sc[2];
        __syncthreads();
        acc = acc / (fmaxf(fabsf(sc[3]), expf(-sc[2])) + A.den_eps);
    }
    if (live && islice == 0) A.out[(size_t)t * A.H * A.dv + (size_t)h * A.dv + jcol] = acc;
}

// How a head of d rows is dealt out: 0: R 4 x IS 8 (d <= 32), 1: 8 x 8 (<= 64), 2: 8 x 16 (<= 128), 3: 8 x 32 (<= 256); -1: too large.
static int scan_shape(int d) { return d <= 32 ? 0 : d <= 64 ? 1 : d <= 128 ? 2 : d <= 256 ? 3 : -1; }

// Floats of state per (head, column slice) for a head of d rows; 0: d is too large.
TL_EXPORT int tl_scan_state_floats(int d, int gated) {
    switch (scan_shape(d)) {
        case 0: return gated ? ScanShape<4, 8, true>::PB : ScanShape<4, 8, false>::PB;
        case 1: return gated ? ScanShape<8, 8, true>::PB : ScanShape<8, 8, false>::PB;
        case 2: return gated ? ScanShape<8, 16, true>::PB : ScanShape<8, 16, false>::PB;
        case 3: return gated ? ScanShape<8, 32, true>::PB : ScanShape<8, 32, false>::PB;
    }
    return 0;
}
TL_EXPORT int tl_scan_columns() { return SCAN_JS; }

template <typename TA, int R, int IS, bool GATED>
static int launch_scan_shape(const ScanArgs& A, int B, bool single, cudaStream_t stream) {
    using Sh = ScanShape<R, IS, GATED>;
    const int nz = (A.dv + SCAN_JS - 1) / SCAN_JS;
    if (single) {
        return launch_after_wait(linear_step_kernel<TA, R, IS, GATED>, dim3(B, A.H, nz), dim3(Sh::NT), 0, stream, A);
    }
    const size_t smem = (size_t)(2 * SCAN_C * Sh::TS + SCAN_C * SCAN_JS + 4 * SCAN_C + A.rot / 2) * sizeof(float);
    if (smem > 48 * 1024) {                              // the widest heads: more dynamic shared memory than a kernel has by default
        static bool raised[TL_MAX_DEVICES] = {};
        const int dev = tl_device_index();
        if (dev < 0) return 1;
        if (!raised[dev]) {
            const cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel<TA, R, IS, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised[dev] = true;
        }
    }
    linear_scan_kernel<TA, R, IS, GATED><<<dim3(B, A.H, nz), Sh::NT, smem, stream>>>(A);
    return tl_launch_status();
}

template <typename TA, bool GATED>
static int launch_scan(const ScanArgs& A, int B, bool single, cudaStream_t stream) {
    switch (scan_shape(A.d)) {
        case 0: return launch_scan_shape<TA, 4, 8, GATED>(A, B, single, stream);
        case 1: return launch_scan_shape<TA, 8, 8, GATED>(A, B, single, stream);
        case 2: return launch_scan_shape<TA, 8, 16, GATED>(A, B, single, stream);
        case 3: return launch_scan_shape<TA, 8, 32, GATED>(A, B, single, stream);
    }
    return 1;
}

TL_EXPORT int tl_linear_scan(const void* proj, int act_dtype, int stride, int q_off, int k_off, int v_off,
                             const float* gates, float cap, const float* decay, const float* inv_freq, int rot,
                             int interleaved, const int* pos, float q_scale, float k_scale, float* state,
                             long long slot_stride, const int* q_start, const int* slots, float* out, int B, int H,
                             int d, int dv, float den_eps, int single_tokens, cudaStream_t stream) {
    // single_tokens: every request of the step brings exactly one token (the caller knows; the step kernel takes it)
    if (B <= 0 || H <= 0) return 0;
    if (H > 65535 || (rot & 1) || rot > d) return 1;
    const ScanArgs A{proj, stride, q_off, k_off, v_off, gates, cap, decay, inv_freq, rot, interleaved, pos, q_scale, k_scale,
                     state, slot_stride, q_start, slots, out, H, d, dv, den_eps};
    const bool gated = gates != nullptr;
    const bool single = single_tokens != 0;
    if (act_dtype == TL_F32) return gated ? launch_scan<float, true>(A, B, single, stream) : launch_scan<float, false>(A, B, single, stream);
    return gated ? launch_scan<bf16, true>(A, B, single, stream) : launch_scan<bf16, false>(A, B, single, stream);
}

// ------------------------------------------------------------------ per-head RMS norm, weight, gate
// out[t, h, j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * (w ? w[h dv + j] : 1) * act(g[t, h dv + j]); one warp per
// (token, head); act 0: no gate, 1: sigmoid, 2: silu.  o is float, out of the activation type, g of its own type (the
// projection that holds the gate may be kept in float).
template <typename TA, typename TW, typename TG>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const TG* __restrict__ g, int g_stride,
                                      const TW* __restrict__ w, TA* __restrict__ out, int H, int dv, float eps, int act) {
    const int t = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
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
            const float x = to_f<TG>(g[(size_t)t * g_stride + h * dv + j]);
            const float s = 1.0f / (1.0f + expf(-x));
            v *= act == 1 ? s : x * s;
        }
        out[((size_t)t * H + h) * dv + j] = from_f<TA>(v);
    }
}

TL_EXPORT int tl_head_norm_gate(const float* o, const void* g, int g_dtype, int g_stride, const void* w, int w_dtype, void* out,
                                int act_dtype, int T, int H, int dv, float eps, int act, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    const dim3 grid(T, (H + 3) / 4), block(128);
#define HNG(TA, TW, TG) launch_after_wait(head_norm_gate_kernel<TA, TW, TG>, grid, block, 0, stream, o, (const TG*)g, g_stride, (const TW*)w, (TA*)out, H, dv, eps, act)
#define HNG_G(TA, TW) { if (g_dtype == TL_F32) HNG(TA, TW, float); else HNG(TA, TW, bf16); }
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) HNG_G(float, float) else HNG_G(float, bf16) }
    else { if (w_dtype == TL_F32) HNG_G(bf16, float) else HNG_G(bf16, bf16) }
#undef HNG_G
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
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
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
#define SN(TA, TW) launch_after_wait(sum_normed_kernel<TA, TW>, dim3(T), dim3(256), 0, stream, (const TA*)a, (const TA*)b, (const TW*)wa, (const TW*)wb, (TA*)out, W, eps, c)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) SN(float, float); else SN(float, bf16); }
    else { if (w_dtype == TL_F32) SN(bf16, float); else SN(bf16, bf16); }
#undef SN
    return tl_launch_status();
}
