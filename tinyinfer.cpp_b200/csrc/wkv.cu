// A recurrent mixer with a decaying matrix state per head (RWKV-style time mixing), and the
// row-wise kernels around it.
//
//  * token_shift_mix: for each of `n_mix` learned vectors mu_s, out[s][t] = h[t] + (h'[t] - h[t])
//    * mu_s, where h'[t] is the row of the token before t in the same request: the row above it
//    in the batch, or, for the first token that a request brings in this step, the row that the
//    request's state kept from its last step (zeros for a new request).
//  * wkv_recurrence: one block per (request, head) walks the request's tokens in order with the
//    head's state S [d keys, d values] (float32, a column per thread, in registers):
//        decay_i = exp(-exp(a_i + w0_i)),  o_j = sum_i r_i (S_ij + u_i k_i v_j),
//        S_ij <- decay_i S_ij + k_i v_j,
//    then brings o to unit root mean square over the head, multiplies by a weight per element and
//    by silu(g) and writes the row; at the end it stores S and (head 0) the last row of h into
//    the request's state slot.
//  * tanh_rows, xielu_rows: float32 in, activation dtype out.
//        xielu(z) = a_p z^2 + z/2 for z > 0, a_q (exp(z) - 1 - z) + z/2 otherwise.
//
// Everything that enters the recurrence is float32: r, k, v, the decay's argument, exponentials,
// the state, the unit norm.  The sum over i runs in ascending order whatever the batch.
#include "common.cuh"

namespace {

template <typename TH>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(const TH* h, const float* __restrict__ mu, int n_mix, int width, int num_tokens,
                       const int* __restrict__ req_of_tok, const int* __restrict__ cu_q,
                       const int* __restrict__ slots, const float* state, size_t state_stride,
                       size_t prev_offset, TH* __restrict__ out) {
    const int t = blockIdx.x;
    const int r = req_of_tok[t];
    const bool first = t == cu_q[r];
    const float* kept = state + (size_t)slots[r] * state_stride + prev_offset;
    const TH* cur = h + (size_t)t * width;
    const TH* above = h + (size_t)(t - (first ? 0 : 1)) * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float x = to_f32(cur[e]);
        const float p = first ? kept[e] : to_f32(above[e]);
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * num_tokens + t) * width + e] = from_f32<TH>(fmaf(p - x, mu[(size_t)s * width + e], x));
    }
}

template <typename TH, typename TO, int DMAX>
__global__ void __launch_bounds__(DMAX)
wkv_recurrence_kernel(const float* r, const float* k, const float* v, const float* g, const float* a,
                      int in_stride, const float* __restrict__ w0, const float* __restrict__ u,
                      const float* __restrict__ norm_weight, float eps, const TH* h, int width,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, float* state,
                      size_t state_stride, size_t prev_offset, int num_heads, int d,
                      TO* __restrict__ out) {
    __shared__ float rs[2][DMAX], ks[2][DMAX], ws[2][DMAX], us[DMAX];
    __shared__ float scratch[32];
    const int req = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int t0 = cu_q[req], t1 = cu_q[req + 1];
    const bool live = j < d;
    float* slot = state + (size_t)slots[req] * state_stride;
    float* s_head = slot + (size_t)head * d * d;
    float S[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = (live && i < d) ? s_head[(size_t)i * d + j] : 0.0f;
    const int col = head * d + j;
    const float w0j = live ? w0[col] : 0.0f, nw = live ? norm_weight[col] : 0.0f;
    us[j] = live ? u[col] : 0.0f;
    for (int t = t0; t < t1; ++t) {
        const int b = (t - t0) & 1;
        const size_t at = (size_t)t * in_stride + col;
        float vj = 0.0f, gj = 0.0f;
        if (live) {
            rs[b][j] = r[at];
            ks[b][j] = k[at];
            ws[b][j] = expf(-expf(a[at] + w0j));
            vj = v[at];
            gj = g[at];
        } else {
            rs[b][j] = 0.0f; ks[b][j] = 0.0f; ws[b][j] = 0.0f;
        }
        __syncthreads();
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < DMAX; ++i) {
            if (i < d) {
                const float kv = ks[b][i] * vj;
                o = fmaf(rs[b][i], fmaf(us[i], kv, S[i]), o);
                S[i] = fmaf(ws[b][i], S[i], kv);
            }
        }
        const float mean = block_sum(live ? o * o : 0.0f, scratch) / (float)d;
        if (live) {
            const float y = o * (1.0f / sqrtf(mean + eps)) * nw * (gj / (1.0f + expf(-gj)));
            out[(size_t)t * num_heads * d + col] = from_f32<TO>(y);
        }
    }
    if (t1 > t0) {
        if (live) {
#pragma unroll
            for (int i = 0; i < DMAX; ++i)
                if (i < d) s_head[(size_t)i * d + j] = S[i];
        }
        if (head == 0) {
            const TH* last = h + (size_t)(t1 - 1) * width;
            for (int e = j; e < width; e += blockDim.x) slot[prev_offset + e] = to_f32(last[e]);
        }
    }
}

template <typename TO>
__global__ void tanh_rows_kernel(const float* x, size_t n, TO* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<TO>(tanhf(x[i]));
}

template <typename TO>
__global__ void xielu_rows_kernel(const float* x, size_t n, float ap, float aq, TO* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = x[i];
    const float y = z > 0.0f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
    out[i] = from_f32<TO>(y);
}

}  // namespace

extern "C" int ti_token_shift_mix(const void* h, int h_dtype, const float* mu, int n_mix, int width,
                                  int num_tokens, const int* req_of_tok, const int* cu_q, const int* slots,
                                  const float* state, long long state_stride, long long prev_offset,
                                  void* out, void* stream) {
    if (num_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == TI_F32)
        token_shift_mix_kernel<float><<<num_tokens, 256, 0, s>>>((const float*)h, mu, n_mix, width, num_tokens,
            req_of_tok, cu_q, slots, state, (size_t)state_stride, (size_t)prev_offset, (float*)out);
    else if (h_dtype == TI_BF16)
        token_shift_mix_kernel<bf16><<<num_tokens, 256, 0, s>>>((const bf16*)h, mu, n_mix, width, num_tokens,
            req_of_tok, cu_q, slots, state, (size_t)state_stride, (size_t)prev_offset, (bf16*)out);
    else
        return ti_fail("token_shift_mix: dtype code %d is not supported", h_dtype);
    return ti_check_launch("token_shift_mix");
}

extern "C" int ti_wkv_recurrence_max_dim() { return 128; }

extern "C" int ti_wkv_recurrence(const float* r, const float* k, const float* v, const float* g, const float* a,
                                 int in_stride, const float* w0, const float* u, const float* norm_weight,
                                 float eps, const void* h, int h_dtype, int width, const int* cu_q,
                                 const int* slots, float* state, long long state_stride, long long prev_offset,
                                 int num_requests, int num_heads, int d, void* out, void* stream) {
    if (num_requests == 0) return 0;
    TI_REQUIRE(d >= 1 && d <= 128, "wkv_recurrence: head size %d must be at most 128", d);
    dim3 grid(num_requests, num_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TH, DMAX)                                                                           \
    wkv_recurrence_kernel<TH, TH, DMAX><<<grid, DMAX, 0, s>>>(                                       \
        r, k, v, g, a, in_stride, w0, u, norm_weight, eps, (const TH*)h, width, cu_q, slots, state,    \
        (size_t)state_stride, (size_t)prev_offset, num_heads, d, (TH*)out)
#define CALL(TH)                                                                                   \
    if (d <= 32) LAUNCH(TH, 32); else if (d <= 64) LAUNCH(TH, 64); else LAUNCH(TH, 128)
    if (h_dtype == TI_F32) { CALL(float); }
    else if (h_dtype == TI_BF16) { CALL(bf16); }
    else return ti_fail("wkv_recurrence: dtype code %d is not supported", h_dtype);
#undef CALL
#undef LAUNCH
    return ti_check_launch("wkv_recurrence");
}

extern "C" int ti_tanh_rows(const float* x, long long n, void* out, int out_dtype, void* stream) {
    if (n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == TI_F32) tanh_rows_kernel<float><<<blocks, 256, 0, s>>>(x, (size_t)n, (float*)out);
    else if (out_dtype == TI_BF16) tanh_rows_kernel<bf16><<<blocks, 256, 0, s>>>(x, (size_t)n, (bf16*)out);
    else return ti_fail("tanh_rows: dtype code %d is not supported", out_dtype);
    return ti_check_launch("tanh_rows");
}

extern "C" int ti_xielu_rows(const float* x, long long n, float ap, float aq, void* out, int out_dtype,
                             void* stream) {
    if (n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == TI_F32) xielu_rows_kernel<float><<<blocks, 256, 0, s>>>(x, (size_t)n, ap, aq, (float*)out);
    else if (out_dtype == TI_BF16) xielu_rows_kernel<bf16><<<blocks, 256, 0, s>>>(x, (size_t)n, ap, aq, (bf16*)out);
    else return ti_fail("xielu_rows: dtype code %d is not supported", out_dtype);
    return ti_check_launch("xielu_rows");
}
