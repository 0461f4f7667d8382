// The gated delta rule with a decay per key channel, and what surrounds it in a mixer: short
// causal convolutions with SiLU on q, k and v, unit-length q and k, the write strength beta, the
// decay, the recurrence itself, and the gated per-head RMS norm of what it reads out.
//
// Per head, with S [D, Dv] (float32, zero when a request starts), for each token in order:
//     S <- g * S            (row d scaled by g_d = exp(-exp(A_log) * softplus(a_d + dt_bias_d)))
//     u  = beta * (v - S^T k)
//     S <- S + k u^T
//     o  = S^T q            (the read-out sees this token's write)
// Everything here is float32: the projections come in as float32, and the state of a request
// (S of every head, then the last taps - 1 inputs of the convolutions) lives in one float32
// vector per request slot.
//
// Four kernels a step:
//   delta_prepare      one block per token, all tokens at once: convolution (the inputs before a
//                      portion's first token come from the slot), SiLU, norms, beta, decay (beta
//                      rides behind each head's decays, so the scan copies both as one row)
//   delta_conv_state   per request: the slot's last taps - 1 inputs after this step
//   delta_scan         per (request, head, group of value columns): the recurrence over the
//                      request's tokens in order.  A thread owns a run of consecutive rows of one
//                      column of S in registers; the R threads of a column add up S^T k and S^T q
//                      by shuffles in a fixed order.  Columns never talk to each other, so the
//                      result does not depend on how a prompt was cut or what else is in the batch.
//   delta_output       per (token, head): o / rms(o) * weight * sigmoid(gate)
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_delta_rule)

namespace {
constexpr int PREP_THREADS = 256;
constexpr int MAX_TAPS = 16;
constexpr int SCAN_THREADS = 128;
constexpr int TCH = 16;           // tokens whose k, q, decay, beta and v a block stages at a time

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// proj columns: q (G D) | k (G D) | v (H Dv) | beta (H) | ...   conv_w: [C, taps], C = 2 G D + H Dv, rows in that order.
// out_c [tokens, C]: q (unit length, times D^-1/2) | k (unit length) | v, after convolution and SiLU.
// gb [tokens, H, D + 4]: per head the D decays, beta, and three zeros.
__global__ void __launch_bounds__(PREP_THREADS) delta_prepare_kernel(
    const float *__restrict__ proj, int ldp, const float *__restrict__ a_pre, int lda, const float *__restrict__ conv_w, int taps,
    const float *__restrict__ state, long long state_stride, long long conv_off, const int *__restrict__ seq_of_token,
    const int *__restrict__ seq_start, const int *__restrict__ slots, const float *__restrict__ a_log,
    const float *__restrict__ dt_bias, float *__restrict__ out_c, float *__restrict__ gb, int H, int G, int D, int Dv) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float buf[];             // the token's C channels after convolution and SiLU
    const int t = blockIdx.x, tid = threadIdx.x;
    const int C = 2 * G * D + H * Dv;
    const int seq = seq_of_token[t];
    const int i = t - seq_start[seq];          // index of the token in its request's portion
    const float *old = state + (size_t)slots[seq] * state_stride + conv_off;   // [(taps - 1), C]: inputs at portion indices -(taps-1) .. -1
    for (int c = tid; c < C; c += PREP_THREADS) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {       // input j tokens back, weighed by column taps - 1 - j
            const int idx = i - j;
            const float x = idx >= 0 ? act_load(proj + (size_t)(t - j) * ldp + c) : act_load(old + (size_t)(taps - 1 + idx) * C + c);
            acc = fmaf(conv_w[(size_t)c * taps + (taps - 1 - j)], x, acc);
        }
        buf[c] = acc * sigmoid_f(acc);
    }
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5;
    float *dst = out_c + (size_t)t * C;
    for (int hd = warp; hd < 2 * G; hd += PREP_THREADS / 32) {       // q heads, then k heads
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(buf[hd * D + d], buf[hd * D + d], ss);
        ss = warp_sum(ss);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        if (hd < G) inv *= 1.0f / sqrtf((float)D);
        for (int d = lane; d < D; d += 32) dst[hd * D + d] = buf[hd * D + d] * inv;
    }
    for (int c = 2 * G * D + tid; c < C; c += PREP_THREADS) dst[c] = buf[c];
    // per head a row of D + 4 floats: the D decays, then beta, then zeros (the row stays a multiple of 16 bytes)
    const int DB = D + 4;
    for (int e = tid; e < H * DB; e += PREP_THREADS) {
        const int h = e / DB, d = e - h * DB;
        float v = 0.f;
        if (d < D) {
            const int c = h * D + d;
            v = expf(-expf(a_log[h]) * softplus_f(act_load(a_pre + (size_t)t * lda + c) + dt_bias[c]));
        } else if (d == D) {
            v = sigmoid_f(act_load(proj + (size_t)t * ldp + C + h));
        }
        gb[(size_t)t * H * DB + e] = v;
    }
}

__global__ void __launch_bounds__(PREP_THREADS) delta_conv_state_kernel(
    const float *__restrict__ proj, int ldp, int taps, float *__restrict__ state, long long state_stride, long long conv_off,
    const int *__restrict__ seq_start, const int *__restrict__ slots, int C) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, c = blockIdx.y * PREP_THREADS + threadIdx.x;
    if (c >= C) return;
    const int t0 = seq_start[s], n = seq_start[s + 1] - t0;
    float *st = state + (size_t)slots[s] * state_stride + conv_off;
    float old[MAX_TAPS];
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r)
        if (r < taps - 1) old[r] = st[(size_t)r * C + c];
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r)
        if (r < taps - 1) {
            const int idx = n - (taps - 1) + r;     // the portion's index that row r holds after this step
            st[(size_t)r * C + c] = idx >= 0 ? act_load(proj + (size_t)(t0 + idx) * ldp + c) : old[taps - 1 + idx];
        }
}

__device__ __forceinline__ void cp_async_16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NPT consecutive rows (d = r NPT .. r NPT + NPT - 1) of one column of S per thread; R threads (a
// power of two, neighbours in a warp) per column.  A block stages TCH tokens at a time in shared
// memory: k, q (thread r's NPT values at floats r (NPT + 4) ..., read as 16-byte pieces; the four
// floats between two threads' runs keep those reads off each other's banks; rows past D hold 0),
// the decays laid out alike with beta behind them (decays past D hold 1) and its value columns.  ASYNC (sizes that are multiples of 4 floats): two such buffers, the next chunk copied
// with cp.async (through L2) while this one is computed; else one buffer filled with plain loads.
// NC columns a thread (column c of a thread lies SCAN_THREADS / R columns after its column c - 1):
// two independent chains per thread fill the waits of each other, and k, q and the decays are read once for both.
template <int NPT, bool ASYNC, int NC>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(
    const float *__restrict__ qkv_c, const float *__restrict__ gb, float *__restrict__ state, long long state_stride,
    const int *__restrict__ seq_start, const int *__restrict__ slots, float *__restrict__ o_out, int H, int G, int D, int Dv, int R) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int RUN = NPT + 4;                          // floats from one thread's run to the next
    const int DP = RUN * R;
    const int DB = D + 4, GP = DP + 4;
    const int tcols = SCAN_THREADS / R;                   // columns side by side in a block; a thread's columns lie tcols apart
    const int cols = NC * tcols;
    const int buf_floats = TCH * (2 * DP + GP + cols);
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int g = h / (H / G);
    const int r = tid % R, col_local = tid / R;
    const int col0 = blockIdx.z * cols;
    const int C = 2 * G * D + H * Dv;
    const int t0 = seq_start[s], n = seq_start[s + 1] - t0;
    float *S_base = state + (size_t)slots[s] * state_stride + (size_t)h * D * Dv;

    float S[NC][NPT];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int d = r * NPT + i, col = col0 + col_local + c * tcols;
            S[c][i] = (col < Dv && d < D) ? S_base[(size_t)d * Dv + col] : 0.f;
        }
    // what the copies never write: rows past D (a decay of 1 and a key of 0 leave them alone), columns
    // past Dv; only the token rows and the buffers this launch will use (a decode step has one token)
    {
        const int rows = min(n, TCH), nb = (ASYNC && n > TCH) ? 2 : 1;
        for (int b = 0; b < nb; ++b) {
            float *k_s = sm + b * buf_floats, *q_s = k_s + TCH * DP, *g_s = q_s + TCH * DP, *v_s = g_s + TCH * GP;
            for (int e = tid; e < rows * DP; e += SCAN_THREADS) k_s[e] = q_s[e] = 0.f;
            for (int e = tid; e < rows * GP; e += SCAN_THREADS) g_s[e] = (e % GP) < DP ? 1.f : 0.f;
            for (int e = tid; e < rows * cols; e += SCAN_THREADS) v_s[e] = 0.f;
        }
    }
    __syncthreads();

    auto stage = [&](int c0, float *buf) {
        const int nt = min(TCH, n - c0);
        float *k_s = buf, *q_s = k_s + TCH * DP, *g_s = q_s + TCH * DP, *v_s = g_s + TCH * GP;
        if (ASYNC) {
            const int d4 = D / 4, b4 = DB / 4, c4 = cols / 4;
            for (int e = tid; e < nt * d4; e += SCAN_THREADS) {
                const int i = e / d4, d = (e - i * d4) * 4;
                const float *row = qkv_c + (size_t)(t0 + c0 + i) * C + g * D + d;
                const int at = (d / NPT) * RUN + d % NPT;          // row d in its thread's run
                cp_async_16(q_s + i * DP + at, row);
                cp_async_16(k_s + i * DP + at, row + G * D);
            }
            for (int e = tid; e < nt * b4; e += SCAN_THREADS) {
                const int i = e / b4, d = (e - i * b4) * 4;
                // the decays go to their places, beta (the row's last four floats) behind the padded row
                cp_async_16(g_s + i * GP + (d < D ? (d / NPT) * RUN + d % NPT : DP), gb + ((size_t)(t0 + c0 + i) * H + h) * DB + d);
            }
            for (int e = tid; e < nt * c4; e += SCAN_THREADS) {
                const int i = e / c4, cl = (e - i * c4) * 4;
                if (col0 + cl < Dv) cp_async_16(v_s + i * cols + cl, qkv_c + (size_t)(t0 + c0 + i) * C + 2 * G * D + h * Dv + col0 + cl);
            }
        } else {
            for (int e = tid; e < nt * D; e += SCAN_THREADS) {
                const int i = e / D, d = e - i * D;
                const float *row = qkv_c + (size_t)(t0 + c0 + i) * C + g * D + d;
                const int at = (d / NPT) * RUN + d % NPT;
                q_s[i * DP + at] = act_load(row);
                k_s[i * DP + at] = act_load(row + G * D);
            }
            for (int e = tid; e < nt * (D + 1); e += SCAN_THREADS) {
                const int i = e / (D + 1), d = e - i * (D + 1);
                g_s[i * GP + (d < D ? (d / NPT) * RUN + d % NPT : DP)] = act_load(gb + ((size_t)(t0 + c0 + i) * H + h) * DB + d);
            }
            for (int e = tid; e < nt * cols; e += SCAN_THREADS) {
                const int i = e / cols, cl = e - i * cols;
                if (col0 + cl < Dv) v_s[e] = act_load(qkv_c + (size_t)(t0 + c0 + i) * C + 2 * G * D + h * Dv + col0 + cl);
            }
        }
    };

    if (ASYNC) {
        stage(0, sm);
        cp_async_commit();
    }
    int turn = 0;
    for (int c0 = 0; c0 < n; c0 += TCH, ++turn) {
        const int nt = min(TCH, n - c0);
        float *buf = sm + (ASYNC ? (turn & 1) * buf_floats : 0);
        if (ASYNC) {
            if (c0 + TCH < n) stage(c0 + TCH, sm + ((turn + 1) & 1) * buf_floats);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            stage(c0, buf);
        }
        __syncthreads();
        const float *k_s = buf, *q_s = k_s + TCH * DP, *g_s = q_s + TCH * DP, *v_s = g_s + TCH * GP;
        for (int i = 0; i < nt; ++i) {
            // this thread's runs of k, q and the decays, in registers by 16-byte reads
            float kk[NPT], qq[NPT], gg[NPT];
#pragma unroll
            for (int j = 0; j < NPT; j += 4) {
                *reinterpret_cast<float4 *>(kk + j) = *reinterpret_cast<const float4 *>(k_s + i * DP + r * RUN + j);
                *reinterpret_cast<float4 *>(gg + j) = *reinterpret_cast<const float4 *>(g_s + i * GP + r * RUN + j);
                *reinterpret_cast<float4 *>(qq + j) = *reinterpret_cast<const float4 *>(q_s + i * DP + r * RUN + j);
            }
            // four partial sums each (NPT is a multiple of 4), added in a fixed order: the chain of
            // dependent operations per token is a quarter as long, and the next token waits on it
            float ks[NC], oq[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float ka[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < NPT; ++j) {
                    S[c][j] *= gg[j];
                    ka[j & 3] = fmaf(kk[j], S[c][j], ka[j & 3]);
                }
                ks[c] = (ka[0] + ka[1]) + (ka[2] + ka[3]);
            }
            for (int o = 1; o < R; o <<= 1)
#pragma unroll
                for (int c = 0; c < NC; ++c) ks[c] += __shfl_xor_sync(0xffffffffu, ks[c], o);
            const float beta = g_s[i * GP + DP];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float u = beta * (v_s[i * cols + col_local + c * tcols] - ks[c]);
                float qa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < NPT; ++j) {
                    S[c][j] = fmaf(kk[j], u, S[c][j]);
                    qa[j & 3] = fmaf(qq[j], S[c][j], qa[j & 3]);
                }
                oq[c] = (qa[0] + qa[1]) + (qa[2] + qa[3]);
            }
            for (int o = 1; o < R; o <<= 1)
#pragma unroll
                for (int c = 0; c < NC; ++c) oq[c] += __shfl_xor_sync(0xffffffffu, oq[c], o);
            if (r == 0) {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int col = col0 + col_local + c * tcols;
                    if (col < Dv) o_out[(size_t)(t0 + c0 + i) * H * Dv + (size_t)h * Dv + col] = oq[c];
                }
            }
        }
        __syncthreads();            // the buffer is free for the copy after next
    }
    if (ASYNC) cp_async_wait<0>();
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int d = r * NPT + i, col = col0 + col_local + c * tcols;
            if (col < Dv && d < D) S_base[(size_t)d * Dv + col] = S[c][i];
        }
}

template <typename T>
__global__ void __launch_bounds__(128) delta_output_kernel(const float *__restrict__ o, const float *__restrict__ weight,
                                                           const float *__restrict__ gate, int ldg, T *__restrict__ out, int ldo, int H,
                                                           int Dv, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const float *row = o + ((size_t)t * H + h) * Dv;
    float ss = 0.f;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        const float v = act_load(row + d);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        const float v = act_load(row + d) * inv * weight[d] * sigmoid_f(act_load(gate + (size_t)t * ldg + (size_t)h * Dv + d));
        out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<T>(v);
    }
}

template <int NPT, bool ASYNC, int NC>
int launch_scan(dim3 grid, size_t smem, cudaStream_t stream, const float *qkv_c, const float *gb, float *state, long long state_stride,
                const int *seq_start, const int *slots, float *o_out, int H, int G, int D, int Dv, int R) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<NPT, ASYNC, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("delta_scan: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(delta_scan_kernel<NPT, ASYNC, NC>, grid, SCAN_THREADS, smem, stream, qkv_c, gb, state, state_stride, seq_start, slots, o_out, H, G, D,
                Dv, R);
    return lgml_launch_status("delta_scan");
}
}  // namespace

LGML_API int lgml_delta_prepare(const float *proj, int ldp, const float *a_pre, int lda, const float *conv_w, int taps, float *state,
                                long long state_stride, long long conv_off, const int *seq_of_token, const int *seq_start,
                                const int *slots, const float *a_log, const float *dt_bias, float *out_c, float *gb, int n_tokens,
                                int n_seqs, int H, int G, int D, int Dv, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && n_seqs >= 0 && H > 0 && G > 0 && D > 0 && Dv > 0, "delta_prepare: bad sizes");
    LGML_REQUIRE(H % G == 0, "delta_prepare: %d heads are no multiple of %d key heads", H, G);
    LGML_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "delta_prepare: %d taps (1 to %d)", taps, MAX_TAPS);
    const int C = 2 * G * D + H * Dv;
    LGML_REQUIRE(ldp >= C + H && lda >= H * D, "delta_prepare: a row stride is below its columns");
    LGML_REQUIRE((size_t)C * sizeof(float) <= 48 * 1024, "delta_prepare: %d channels are more than a block's shared memory holds", C);
    if (n_tokens == 0) return 0;
    lgml_launch(delta_prepare_kernel, dim3(n_tokens), PREP_THREADS, (size_t)C * sizeof(float), stream, proj, ldp, a_pre, lda, conv_w, taps,
                (const float *)state, state_stride, conv_off, seq_of_token, seq_start, slots, a_log, dt_bias, out_c, gb, H, G, D, Dv);
    int rc = lgml_launch_status("delta_prepare");
    if (rc || taps == 1) return rc;
    lgml_launch(delta_conv_state_kernel, dim3(n_seqs, (C + PREP_THREADS - 1) / PREP_THREADS), PREP_THREADS, 0, stream, proj, ldp, taps, state,
                state_stride, conv_off, seq_start, slots, C);
    return lgml_launch_status("delta_conv_state");
}

// gb: float32 [tokens, H, D + 4] as delta_prepare writes it (decays, beta, zeros).
LGML_API int lgml_delta_scan(const float *qkv_c, const float *gb, float *state, long long state_stride, const int *seq_start,
                             const int *slots, float *o_out, int n_seqs, int H, int G, int D, int Dv, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && H > 0 && G > 0 && D > 0 && Dv > 0 && H % G == 0, "delta_scan: bad sizes");
    LGML_REQUIRE(D <= 1024, "delta_scan: key size %d is over 1024", D);
    LGML_REQUIRE(H <= 65535, "delta_scan: too many heads");
    if (n_seqs == 0) return 0;
    int R = 1;
    // 16 rows a thread while 32 threads a column suffice.  (More threads a column do not pay although one
    // prompt leaves most warp slots empty: 2,048 tokens of 16 heads of 128 x 128 take 0.97 ms with 8
    // threads a column, 1.02 with 16, 2.36 with 32.  Every block walks the whole chain of tokens, so
    // the blocks must all be resident at once: with 32 such heads, 16 threads a column made 512 blocks
    // where 444 fit, and the prompt took twice as long.)
    while (R < 32 && (D + R - 1) / R > 16) R *= 2;
    const int rows = (D + R - 1) / R;
    const int npt = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    // Two columns a thread where a head has them, a thread's rows are few enough for the registers, and
    // the grid still covers the SMs twice (many requests in a step: 30.8 us against 33.8 for 8 requests of
    // 16 heads of 128 x 128).  One request's prompt is a chain per column, and half as many warps each
    // with two chains were slower there (1.14 ms against 0.97 for 2,048 tokens), so it keeps one.
    const int tcols = SCAN_THREADS / R;
    const bool wide = npt <= 16 && Dv >= 2 * tcols && (long long)n_seqs * H * ((Dv + 2 * tcols - 1) / (2 * tcols)) >= 2 * 148;
    const int nc = wide ? 2 : 1;
    const int cols = nc * (SCAN_THREADS / R);
    const bool async = D % 4 == 0 && Dv % 4 == 0 && (((uintptr_t)qkv_c | (uintptr_t)gb) & 15) == 0;
    const size_t smem = sizeof(float) * (size_t)(async ? 2 : 1) * TCH * (3 * (size_t)(npt + 4) * R + 4 + cols);
    dim3 grid(n_seqs, H, (Dv + cols - 1) / cols);
#define LGML_SCAN_ARGS grid, smem, stream, qkv_c, gb, state, state_stride, seq_start, slots, o_out, H, G, D, Dv, R
#define LGML_SCAN_CASE(N)                                                                                          \
    if (nc == 2) return async ? launch_scan<N, true, 2>(LGML_SCAN_ARGS) : launch_scan<N, false, 2>(LGML_SCAN_ARGS); \
    return async ? launch_scan<N, true, 1>(LGML_SCAN_ARGS) : launch_scan<N, false, 1>(LGML_SCAN_ARGS);
    switch (npt) {
        case 4: LGML_SCAN_CASE(4)
        case 8: LGML_SCAN_CASE(8)
        case 16: LGML_SCAN_CASE(16)
        default: LGML_SCAN_CASE(32)
    }
#undef LGML_SCAN_CASE
#undef LGML_SCAN_ARGS
}

LGML_API int lgml_delta_output(const float *o, const float *weight, const float *gate, int ldg, void *out, int dtype, int ldo,
                               int n_tokens, int H, int Dv, float eps, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Dv > 0 && H <= 65535, "delta_output: bad sizes");
    LGML_REQUIRE(ldg >= H * Dv && ldo >= H * Dv, "delta_output: a row stride is below H Dv");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, H);
    if (dtype == LGML_F32)
        lgml_launch(delta_output_kernel<float>, grid, 128, 0, stream, o, weight, gate, ldg, (float *)out, ldo, H, Dv, eps);
    else if (dtype == LGML_BF16)
        lgml_launch(delta_output_kernel<__nv_bfloat16>, grid, 128, 0, stream, o, weight, gate, ldg, (__nv_bfloat16 *)out, ldo, H, Dv, eps);
    else
        LGML_FAIL("delta_output: unknown type %d", dtype);
    return lgml_launch_status("delta_output");
}
