// A recurrent mixer with a decaying matrix state per head (RWKV-style time mixing), and the
// row-wise kernels around it.
//
//  * token_shift_mix: for each of `n_mix` learned vectors mu_s, out[s][t] = h[t] + (h'[t] - h[t])
//    * mu_s, where h'[t] is the row of the token before t in the same request: the row above it
//    in the batch, or, for the first token that a request brings in this step, the row that the
//    request's state kept from its last step (zeros for a new request).
//  * wkv_recurrence: one block per (request, head) walks the request's tokens in order with the
//    head's state S [d keys, d values] (float32, in registers, a column per four threads):
//        decay_i = exp(-exp(a_i + w0_i)),  o_j = sum_i r_i (S_ij + u_i k_i v_j),
//        S_ij <- decay_i S_ij + k_i v_j,
//    then brings o to unit root mean square over the head, multiplies by a weight per element and
//    by silu(g) and writes the row; at the end it stores S and (head 0) the last row of h into
//    the request's state slot.
//  * tanh_rows, xielu_rows: float32 in, activation dtype out.
//        xielu(z) = a_p z^2 + z/2 for z > 0, a_q (exp(z) - 1 - z) + z/2 otherwise.
//
// Everything that enters the recurrence is float32: r, k, v, the decay's argument, exponentials,
// the state, the unit norm.  The order of the sum over i depends on nothing but d.
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

// Tokens are staged a tile (16 or 8) at a time: all threads fetch the tile's r, k, v, g and decays into shared
// memory (the next tile's values are already in registers while this one is worked on), then the
// tile's tokens follow one another without a barrier: column j of the state belongs to four
// neighbouring lanes, lane part s holding its rows s, s + 4, s + 8, ...; the four partial sums of
// o_j meet through two shuffles.  The unit norm of the tile's rows is taken afterwards, a warp per
// token.
constexpr int WKV_IS = 4;

template <typename TH, typename TO, int DMAX>
__global__ void __launch_bounds__(DMAX * WKV_IS)
wkv_recurrence_kernel(const float* r, const float* k, const float* v, const float* g, const float* a,
                      int in_stride, const float* __restrict__ w0, const float* __restrict__ u,
                      const float* __restrict__ norm_weight, float eps, const TH* h, int width,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, float* state,
                      size_t state_stride, size_t prev_offset, int num_heads, int d,
                      TO* __restrict__ out) {
    constexpr int WKV_TT = DMAX > 64 ? 8 : 16;           // tokens per staged tile (48 KB of shared memory at most)
    constexpr int NI = DMAX / WKV_IS;                    // state rows per thread
    constexpr int THREADS = DMAX * WKV_IS;
    constexpr int PER = WKV_TT * DMAX / THREADS;         // staged elements of one array per thread
    __shared__ __align__(16) float rs[WKV_TT][DMAX], ks[WKV_TT][DMAX], ws[WKV_TT][DMAX];
    __shared__ float vs[WKV_TT][DMAX], gs[WKV_TT][DMAX], os[WKV_TT][DMAX], us[DMAX], inv_s[WKV_TT];
    const int req = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int j = tid / WKV_IS, part = tid % WKV_IS;
    const int t0 = cu_q[req], t1 = cu_q[req + 1];
    const bool live = j < d;
    float* slot = state + (size_t)slots[req] * state_stride;
    float* s_head = slot + (size_t)head * d * d;
    float S[NI];
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = part + WKV_IS * ii;
        S[ii] = (live && i < d) ? s_head[(size_t)i * d + j] : 0.0f;
    }
    if (tid < DMAX) us[tid] = tid < d ? u[head * d + tid] : 0.0f;

    float fr[PER], fk[PER], fa[PER], fv[PER], fg[PER];
    auto fetch = [&](int tile0) {                        // the tile's values into registers
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            const int e = tid + x * THREADS, tt = e / DMAX, c = e % DMAX;
            const bool ok = tile0 + tt < t1 && c < d;
            const size_t at = (size_t)(tile0 + tt) * in_stride + head * d + c;
            fr[x] = ok ? r[at] : 0.0f;
            fk[x] = ok ? k[at] : 0.0f;
            fa[x] = ok ? a[at] + w0[head * d + c] : 0.0f;
            fv[x] = ok ? v[at] : 0.0f;
            fg[x] = ok ? g[at] : 0.0f;
        }
    };
    if (t0 < t1) fetch(t0);
    for (int tile0 = t0; tile0 < t1; tile0 += WKV_TT) {
        __syncthreads();                                 // the tile before has been read and written out
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            const int e = tid + x * THREADS, tt = e / DMAX, c = e % DMAX;
            rs[tt][c] = fr[x];
            ks[tt][c] = fk[x];
            ws[tt][c] = expf(-expf(fa[x]));
            vs[tt][c] = fv[x];
            gs[tt][c] = fg[x];
        }
        __syncthreads();
        if (tile0 + WKV_TT < t1) fetch(tile0 + WKV_TT);  // in flight while this tile is worked on
        const int nt = min(WKV_TT, t1 - tile0);
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = vs[tt][j];
            float o = 0.0f;
#pragma unroll
            for (int ii = 0; ii < NI; ++ii) {
                const int i = part + WKV_IS * ii;
                const float kv = ks[tt][i] * vj;
                o = fmaf(rs[tt][i], fmaf(us[i], kv, S[ii]), o);
                S[ii] = fmaf(ws[tt][i], S[ii], kv);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (part == 0) os[tt][j] = live ? o : 0.0f;
        }
        __syncthreads();
        for (int tt = tid / 32; tt < nt; tt += THREADS / 32) {       // a warp per token: its unit norm
            float ss = 0.0f;
            for (int c = tid % 32; c < d; c += 32) ss = fmaf(os[tt][c], os[tt][c], ss);
            ss = warp_sum(ss);
            if (tid % 32 == 0) inv_s[tt] = 1.0f / sqrtf(ss / (float)d + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * DMAX; e += THREADS) {
            const int tt = e / DMAX, c = e % DMAX;
            if (c < d) {
                const float gj = gs[tt][c];
                const float y = os[tt][c] * inv_s[tt] * norm_weight[head * d + c] * (gj / (1.0f + expf(-gj)));
                out[(size_t)(tile0 + tt) * num_heads * d + head * d + c] = from_f32<TO>(y);
            }
        }
    }
    if (t1 > t0) {
        if (live) {
#pragma unroll
            for (int ii = 0; ii < NI; ++ii) {
                const int i = part + WKV_IS * ii;
                if (i < d) s_head[(size_t)i * d + j] = S[ii];
            }
        }
        if (head == 0) {
            const TH* last = h + (size_t)(t1 - 1) * width;
            for (int e = tid; e < width; e += THREADS) slot[prev_offset + e] = to_f32(last[e]);
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
    wkv_recurrence_kernel<TH, TH, DMAX><<<grid, DMAX * WKV_IS, 0, s>>>(                                       \
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
