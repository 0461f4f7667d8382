// Attention with a sink, a distance bias and a window over the paged cache, for mixers whose
// keys and values have head sizes of their own (D for q and k, Dv for v).
//
//   score(i, j) = (q_i . k_j) * scale - slope_h * (i - j)        for 0 <= i - j < window (0: all j <= i)
//   weight(i, j) = exp(score(i, j)) / (exp(sink_h) + sum_j' exp(score(i, j')))
//   out_i = sum_j weight(i, j) v_j      [* sigmoid(gate_i) element by element, when a gate is given]
//
// The sink is one more term of the denominator: it has no key and no value.  Scores, the running
// maximum, the sums and the gate are float32 in both compute types.
//
// Two kernels.  sink_qkv_store takes the fused projection's float32 output (q | k | v [| more]),
// multiplies q by its position's temperature 1 + coef * ln(floor((p + 1) / every) + 1), mixes v
// with the values another layer kept for the same token (v <- (1 - lambda) v + lambda v_first), and
// stores k and the mixed v in their cells and q in its own buffer.  sink_attention is the general
// form: one block per (token, head); a (token, head)'s result depends only on that token's
// position and its request's cells, read in a fixed order, so it is the same however the tokens
// were cut into steps and whatever else is in the batch.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_sink)

namespace {
constexpr int ITEMS = 256;
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

// v_mode: 0 store v as it is; 1 also keep it in v_keep (float32 [tokens, Hkv Dv]); 2 mix with v_keep first
template <typename T>
__global__ void __launch_bounds__(ITEMS) sink_qkv_store_kernel(
    const float *__restrict__ proj, int ldp, T *__restrict__ q_out, int ldq, const int *__restrict__ positions,
    const int *__restrict__ seq_of_token, const int *__restrict__ block_table, int max_blocks, T *__restrict__ k_pages,
    T *__restrict__ v_pages, int n_pages, int page_size, int H, int Hkv, int D, int Dv, float temp_coef, int temp_every,
    int v_mode, float *__restrict__ v_keep, const float *__restrict__ v_lambda, int write_kv, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int nq = H * D, nk = Hkv * D, nv = Hkv * Dv;
    const int e = blockIdx.y * ITEMS + threadIdx.x;
    if (e >= nq + (write_kv ? nk + nv : 0)) return;
    const int pos = positions[t];
    float val = act_load(proj + (size_t)t * ldp + e);
    if (e < nq) {
        if (temp_coef != 0.f) val *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
        q_out[(size_t)t * ldq + e] = from_f32<T>(val);
        return;
    }
    const int seq = seq_of_token[t];
    const int blk = pos / page_size;
    int page = -1;
    if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
    if (page < 0 || page >= n_pages) {   // the host reserves pages first; never write outside the pool
        if (e == nq) atomicExch(status, 2);
        return;
    }
    if (e < nq + nk) {
        const int c = e - nq, g = c / D, d = c - g * D;
        k_pages[(((size_t)page * Hkv + g) * page_size + (size_t)(pos % page_size)) * D + d] = from_f32<T>(val);
        return;
    }
    const int c = e - nq - nk, g = c / Dv, d = c - g * Dv;
    if (v_mode == 1) {
        v_keep[(size_t)t * nv + c] = val;
    } else if (v_mode == 2) {
        const float lam = v_lambda[0];
        val = (1.0f - lam) * val + lam * act_load(v_keep + (size_t)t * nv + c);
    }
    v_pages[(((size_t)page * Hkv + g) * page_size + (size_t)(pos % page_size)) * Dv + d] = from_f32<T>(val);
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) sink_attention_kernel(
    const T *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const T *__restrict__ k_pages, const T *__restrict__ v_pages,
    int n_pages, int page_size, const float *__restrict__ slopes, const float *__restrict__ sinks,
    const float *__restrict__ gate, int ldg, T *__restrict__ out, int ldo, int H, int Hkv, int D, int Dv, float scale,
    int window, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float qs[MAX_D];
    __shared__ float acc_w[WARPS][MAX_D];
    __shared__ float m_w[WARPS], l_w[WARPS];
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int *table = block_table + (size_t)seq * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const float slope = slopes ? slopes[h] : 0.f;

    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = to_f32(act_load(q + (size_t)t * ldq + (size_t)h * D + d));
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

    for (int j = lo + warp; j <= pos; j += WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? table[blk] : -1;
        if (page < 0 || page >= n_pages) {  // a cell the table does not hold: flag it, skip the key
            if (lane == 0) atomicExch(status, 3);
            continue;
        }
        const size_t cell = ((size_t)page * Hkv + g) * page_size + (size_t)(j % page_size);
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) dot = fmaf(qs[d], to_f32(act_load(k_pages + cell * D + d)), dot);
        const float s = warp_sum(dot) * scale - slope * (float)(pos - j);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < Dv) acc[i] = acc[i] * corr + p * to_f32(act_load(v_pages + cell * Dv + d));
        }
        m = m_new;
    }
    if (lane == 0) {
        m_w[warp] = m;
        l_w[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc_w[warp][d] = acc[i];
    }
    __syncthreads();
    const float sink = sinks ? sinks[h] : -INFINITY;
    float mm = sink;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, m_w[w]);
    float lsum = sinks ? expf(sink - mm) : 0.f;
    float f[WARPS];
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (m_w[w] == -INFINITY) ? 0.f : expf(m_w[w] - mm);
        lsum += l_w[w] * f[w];
    }
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; ++w) o += acc_w[w][d] * f[w];
        o = lsum > 0.f ? o / lsum : 0.f;
        if (gate) o *= 1.0f / (1.0f + expf(-act_load(gate + (size_t)t * ldg + (size_t)h * Dv + d)));
        out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<T>(o);
    }
}
}  // namespace

// proj: float32 [n_tokens, ldp], columns q (H D) | k (Hkv D) | v (Hkv Dv) | anything else.
// v_keep: float32 [n_tokens, Hkv Dv], written (v_mode 1) or read (v_mode 2); v_lambda: one float32 on the device.
LGML_API int lgml_sink_qkv_store(const float *proj, int ldp, void *q_out, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                 const int *block_table, int max_blocks, void *k_pages, void *v_pages, int n_pages, int page_size,
                                 int n_tokens, int H, int Hkv, int D, int Dv, float temp_coef, int temp_every, int v_mode, float *v_keep,
                                 const float *v_lambda, int write_kv, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && Dv > 0 && page_size > 0 && max_blocks > 0, "sink_qkv_store: bad sizes");
    LGML_REQUIRE(ldp >= H * D + Hkv * (D + Dv), "sink_qkv_store: row stride %d is below the q, k and v columns", ldp);
    LGML_REQUIRE(ldq >= H * D, "sink_qkv_store: q row stride %d is below H D = %d", ldq, H * D);
    LGML_REQUIRE(temp_coef == 0.f || temp_every > 0, "sink_qkv_store: the temperature's step must be positive");
    LGML_REQUIRE(v_mode >= 0 && v_mode <= 2, "sink_qkv_store: unknown value mode %d", v_mode);
    LGML_REQUIRE(v_mode == 0 || v_keep != nullptr, "sink_qkv_store: value mode %d needs the kept values", v_mode);
    LGML_REQUIRE(v_mode != 2 || v_lambda != nullptr, "sink_qkv_store: mixing needs its weight");
    if (n_tokens == 0) return 0;
    const int items = H * D + (write_kv ? Hkv * (D + Dv) : 0);
    dim3 grid(n_tokens, (items + ITEMS - 1) / ITEMS);
    if (dtype == LGML_F32)
        lgml_launch(sink_qkv_store_kernel<float>, grid, ITEMS, 0, stream, proj, ldp, (float *)q_out, ldq, positions, seq_of_token, block_table,
                    max_blocks, (float *)k_pages, (float *)v_pages, n_pages, page_size, H, Hkv, D, Dv, temp_coef, temp_every, v_mode, v_keep,
                    v_lambda, write_kv, status);
    else if (dtype == LGML_BF16)
        lgml_launch(sink_qkv_store_kernel<__nv_bfloat16>, grid, ITEMS, 0, stream, proj, ldp, (__nv_bfloat16 *)q_out, ldq, positions, seq_of_token,
                    block_table, max_blocks, (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, n_pages, page_size, H, Hkv, D, Dv, temp_coef,
                    temp_every, v_mode, v_keep, v_lambda, write_kv, status);
    else
        LGML_FAIL("sink_qkv_store: unknown type %d", dtype);
    return lgml_launch_status("sink_qkv_store");
}

// slopes, sinks: float32 [H] or null (no bias, no sink); gate: float32 [n_tokens, ldg] (column h Dv + d) or null.
LGML_API int lgml_sink_attention(const void *q, int dtype, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
                                 int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, const float *slopes,
                                 const float *sinks, const float *gate, int ldg, void *out, int ldo, int n_tokens, int H, int Hkv, int D,
                                 int Dv, float scale, int window, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && Dv > 0 && page_size > 0 && max_blocks > 0, "sink_attention: bad sizes");
    LGML_REQUIRE(H % Hkv == 0, "sink_attention: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D <= MAX_D && Dv <= MAX_D, "sink_attention: head sizes %d and %d must be at most %d", D, Dv, MAX_D);
    LGML_REQUIRE(H <= 65535, "sink_attention: too many heads");
    LGML_REQUIRE(window >= 0, "sink_attention: bad window");
    LGML_REQUIRE(gate == nullptr || ldg >= H * Dv, "sink_attention: the gate's row stride %d is below H Dv", ldg);
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, H);
    if (dtype == LGML_F32)
        lgml_launch(sink_attention_kernel<float>, grid, WARPS * 32, 0, stream, (const float *)q, ldq, positions, seq_of_token, block_table,
                    max_blocks, (const float *)k_pages, (const float *)v_pages, n_pages, page_size, slopes, sinks, gate, ldg, (float *)out, ldo, H,
                    Hkv, D, Dv, scale, window, status);
    else if (dtype == LGML_BF16)
        lgml_launch(sink_attention_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, stream, (const __nv_bfloat16 *)q, ldq, positions, seq_of_token,
                    block_table, max_blocks, (const __nv_bfloat16 *)k_pages, (const __nv_bfloat16 *)v_pages, n_pages, page_size, slopes, sinks,
                    gate, ldg, (__nv_bfloat16 *)out, ldo, H, Hkv, D, Dv, scale, window, status);
    else
        LGML_FAIL("sink_attention: unknown type %d", dtype);
    return lgml_launch_status("sink_attention");
}
