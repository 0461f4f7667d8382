// A mixture of experts as a feed-forward: a router picks `top` of X small gated feed-forward
// layers per token; the token's output is the weighted sum of theirs.
//
//   z      = W_r h + b_r                              float32, X logits per token
//   chosen = the `top` largest z (ties: the lower index), w = softmax over the chosen z alone
//   y      = sum_e w_e W_down[e] (silu(W_gate[e] h) * (W_up[e] h))
//
// moe_router writes the chosen experts and their weights, [tokens, top] each.  The experts'
// matrices lie stacked, [X, F, E] for gate and up and [X, E, F] for down.
//
// Two forms of the experts' products.  The row form (moe_gate_up, moe_down): a block per (token,
// chosen expert), a warp per output feature, k in a fixed order; it reads an expert's matrices
// once per token that chose it, which is what a decode step needs and no more, and it is the
// 32-bit path.  The grouped form for many tokens is further down.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_moe)

namespace {

template <typename T>
__global__ void __launch_bounds__(128) moe_router_kernel(const T *__restrict__ h, int ldh, const float *__restrict__ wr, const float *__restrict__ br,
                                                         int *__restrict__ ids, float *__restrict__ wts, int E, int X, int top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float z[];        // X logits
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const T *row = h + (size_t)t * ldh;
    for (int e = warp; e < X; e += n_warps) {
        float dot = 0.f;
        for (int k = lane; k < E; k += 32) dot = fmaf(to_f32(act_load(row + k)), wr[(size_t)e * E + k], dot);
        dot = warp_sum(dot);
        if (lane == 0) z[e] = dot + (br ? br[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    float zmax = 0.f, sum = 0.f;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < X; e += 32) {
            const float v = z[e];
            if (v > best) best = v, at = e;         // strictly greater: a lane keeps its lowest index
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
        }
        if (at == 0x7fffffff) at = 0;               // every logit was -inf or NaN
        if (s == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == 0) {
            ids[(size_t)t * top + s] = at;
            wts[(size_t)t * top + s] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int s = lane; s < top; s += 32) wts[(size_t)t * top + s] *= inv;
}

// act[(t top + s), f] = silu(Wg[e] h_t)[f] * (Wu[e] h_t)[f], e = ids[t, s]
constexpr int GU_WARPS = 4, GU_PER_WARP = 8;
template <typename T>
__global__ void __launch_bounds__(GU_WARPS * 32) moe_gate_up_kernel(const T *__restrict__ h, int ldh, const int *__restrict__ ids, const T *__restrict__ wg,
                                                                    const T *__restrict__ wu, T *__restrict__ act, int E, int F, int X, int top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float hs[];       // the token's row
    const int row = blockIdx.x, t = row / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < E; k += blockDim.x) hs[k] = to_f32(act_load(h + (size_t)t * ldh + k));
    int e = ids[row];
    e = e < 0 ? 0 : (e >= X ? X - 1 : e);
    __syncthreads();
    const int f0 = (blockIdx.y * GU_WARPS + warp) * GU_PER_WARP;
    for (int f = f0; f < f0 + GU_PER_WARP && f < F; ++f) {
        const T *g_row = wg + ((size_t)e * F + f) * E, *u_row = wu + ((size_t)e * F + f) * E;
        float g = 0.f, u = 0.f;
        for (int k = lane; k < E; k += 32) {
            const float x = hs[k];
            g = fmaf(x, to_f32(g_row[k]), g);
            u = fmaf(x, to_f32(u_row[k]), u);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) act[(size_t)row * F + f] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// out[t, j] = sum_s wts[t, s] (Wd[ids[t, s]] act[t top + s])[j], float32; the chosen experts in their order
constexpr int DN_WARPS = 4, DN_PER_WARP = 8;
template <typename T>
__global__ void __launch_bounds__(DN_WARPS * 32) moe_down_kernel(const T *__restrict__ act, const int *__restrict__ ids, const float *__restrict__ wts,
                                                                 const T *__restrict__ wd, float *__restrict__ out, int E, int F, int X, int top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float as[];       // top rows of F
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < top * F; k += blockDim.x) as[k] = to_f32(act_load(act + (size_t)t * top * F + k));
    __syncthreads();
    const int j0 = (blockIdx.y * DN_WARPS + warp) * DN_PER_WARP;
    for (int j = j0; j < j0 + DN_PER_WARP && j < E; ++j) {
        float total = 0.f;
        for (int s = 0; s < top; ++s) {
            int e = ids[(size_t)t * top + s];
            e = e < 0 ? 0 : (e >= X ? X - 1 : e);
            const T *d_row = wd + ((size_t)e * E + j) * F;
            float dot = 0.f;
            for (int k = lane; k < F; k += 32) dot = fmaf(as[(size_t)s * F + k], to_f32(d_row[k]), dot);
            total = fmaf(act_load(wts + (size_t)t * top + s), warp_sum(dot), total);
        }
        if (lane == 0) out[(size_t)t * E + j] = total;
    }
}

template <typename K>
static int need_smem(K kernel, size_t smem, const char *who) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("%s: cannot have %zu bytes of shared memory: %s", who, smem, cudaGetErrorString(e));
    }
    return 0;
}
}  // namespace

// h: [n, ldh] in the compute type; wr: float32 [X, E]; br: float32 [X] or null; ids int32 / wts float32 [n, top]
LGML_API int lgml_moe_router(const void *h, int dtype, int ldh, const float *wr, const float *br, int *ids, float *wts, int n_tokens, int E, int X,
                             int top, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && X > 0 && top > 0 && top <= X, "moe_router: bad sizes (%d experts, %d chosen)", X, top);
    LGML_REQUIRE(X <= 8192, "moe_router: at most 8192 experts");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * (size_t)X;
    if (dtype == LGML_F32)
        lgml_launch(moe_router_kernel<float>, n_tokens, 128, smem, stream, (const float *)h, ldh, wr, br, ids, wts, E, X, top);
    else if (dtype == LGML_BF16)
        lgml_launch(moe_router_kernel<__nv_bfloat16>, n_tokens, 128, smem, stream, (const __nv_bfloat16 *)h, ldh, wr, br, ids, wts, E, X, top);
    else
        LGML_FAIL("moe_router: unknown type %d", dtype);
    return lgml_launch_status("moe_router");
}

// The row form: act [n top, F] in the compute type (scratch of the caller), out float32 [n, E].
LGML_API int lgml_moe_experts_rows(const void *h, int dtype, int ldh, const int *ids, const float *wts, const void *wg, const void *wu, const void *wd,
                                   void *act, float *out, int n_tokens, int E, int F, int X, int top, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && F > 0 && X > 0 && top > 0, "moe_experts_rows: bad sizes");
    if (n_tokens == 0) return 0;
    const size_t smem_gu = sizeof(float) * (size_t)E, smem_dn = sizeof(float) * (size_t)top * F;
    LGML_REQUIRE(smem_gu <= 200 * 1024 && smem_dn <= 200 * 1024, "moe_experts_rows: rows of %d or %d x %d floats do not fit shared memory", E, top, F);
    dim3 grid_gu(n_tokens * top, (F + GU_WARPS * GU_PER_WARP - 1) / (GU_WARPS * GU_PER_WARP));
    dim3 grid_dn(n_tokens, (E + DN_WARPS * DN_PER_WARP - 1) / (DN_WARPS * DN_PER_WARP));
    if (dtype == LGML_F32) {
        if (need_smem(moe_gate_up_kernel<float>, smem_gu, "moe_experts_rows") || need_smem(moe_down_kernel<float>, smem_dn, "moe_experts_rows")) return -1;
        lgml_launch(moe_gate_up_kernel<float>, grid_gu, GU_WARPS * 32, smem_gu, stream, (const float *)h, ldh, ids, (const float *)wg, (const float *)wu,
                    (float *)act, E, F, X, top);
        lgml_launch(moe_down_kernel<float>, grid_dn, DN_WARPS * 32, smem_dn, stream, (const float *)act, ids, wts, (const float *)wd, out, E, F, X, top);
    } else if (dtype == LGML_BF16) {
        if (need_smem(moe_gate_up_kernel<__nv_bfloat16>, smem_gu, "moe_experts_rows") ||
            need_smem(moe_down_kernel<__nv_bfloat16>, smem_dn, "moe_experts_rows"))
            return -1;
        lgml_launch(moe_gate_up_kernel<__nv_bfloat16>, grid_gu, GU_WARPS * 32, smem_gu, stream, (const __nv_bfloat16 *)h, ldh, ids,
                    (const __nv_bfloat16 *)wg, (const __nv_bfloat16 *)wu, (__nv_bfloat16 *)act, E, F, X, top);
        lgml_launch(moe_down_kernel<__nv_bfloat16>, grid_dn, DN_WARPS * 32, smem_dn, stream, (const __nv_bfloat16 *)act, ids, wts,
                    (const __nv_bfloat16 *)wd, out, E, F, X, top);
    } else {
        LGML_FAIL("moe_experts_rows: unknown type %d", dtype);
    }
    return lgml_launch_status("moe_experts_rows");
}
