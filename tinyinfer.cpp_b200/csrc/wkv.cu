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

// Tokens are staged a tile (16 or 8) at a time: cp.async brings the tile's r, k, v, g and decay arguments
// into one of two buffers in shared memory while the tile before is worked on, then
// the tile's tokens follow one another without a barrier: column j of the state belongs to four
// neighbouring lanes (sixteen in the column-split form), each holding its share of the rows (read four
// at a time); their partial sums of o_j meet through shuffles once per tile.  The unit norm of the tile's rows is taken afterwards, a warp per
// token.  JS > 1 (long portions of few requests): a head's columns are cut over JS blocks, each with
// the whole of r, k and the decays and its own columns of v; the blocks write o as float32 and a
// second launch (wkv_finish) takes the norm, the weight and the gate.
// lanes per state column: four, or, where a head's columns are cut over blocks (long portions), up to
// sixteen, so that a token's chain of multiply-adds is a quarter as long
constexpr int wkv_lanes(int dmax, int js) { return js == 1 ? 4 : (dmax / 4 < 16 ? dmax / 4 : 16); }

__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 4 : 0;                     // nothing is read and zero is written otherwise
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

template <typename TH, typename TO, int DMAX, int JS>
__global__ void __launch_bounds__(DMAX / JS * wkv_lanes(DMAX, JS))
wkv_recurrence_kernel(const float* r, const float* k, const float* v, const float* g, const float* a,
                      int in_stride, const float* __restrict__ w0, const float* __restrict__ u,
                      const float* __restrict__ norm_weight, float eps, const TH* h, int width,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, float* state,
                      size_t state_stride, size_t prev_offset, int num_heads, int d,
                      TO* __restrict__ out, float* __restrict__ o_raw) {
    constexpr int WKV_TT = (DMAX > 64 ? 8 : 16) / (JS == 1 ? 2 : 1);   // tokens per staged tile (48 KB of shared memory at most)
    constexpr int WKV_IS = wkv_lanes(DMAX, JS);
    constexpr int NI = DMAX / WKV_IS;                    // state rows per thread
    constexpr int DC = DMAX / JS;                        // state columns of this block
    constexpr int THREADS = DC * WKV_IS;
    constexpr int PER = WKV_TT * DMAX / THREADS;         // staged elements of r, k, decay per thread
    constexpr int PERC = (WKV_TT * DC + THREADS - 1) / THREADS;   // ... of v and g (this block's columns)
    // two buffers of a tile's inputs: one is read while cp.async fills the other
    __shared__ __align__(16) float rs[2][WKV_TT][DMAX], ks[2][WKV_TT][DMAX], as[2][WKV_TT][DMAX], ws[WKV_TT][DMAX];
    __shared__ float vs[2][WKV_TT][DC], gs[2][WKV_TT][DC], os[WKV_TT][DC], inv_s[WKV_TT];
    const int req = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int c0 = blockIdx.z * DC;                      // first column of this block
    const int j = c0 + tid / WKV_IS, part = tid % WKV_IS;
    const int t0 = cu_q[req], t1 = cu_q[req + 1];
    const bool live = j < d;
    float* slot = state + (size_t)slots[req] * state_stride;
    float* s_head = slot + (size_t)head * d * d;
    // lane part `part` has rows 4 IS q + 4 part + x (x = 0..3, q = 0..NI/4 - 1) of column j and their
    // bonus u: the lanes of a column read contiguous bytes of a token's r, k or decay, four rows each
    float S[NI], ur[NI];
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = (ii / 4) * (4 * WKV_IS) + part * 4 + ii % 4;
        S[ii] = (live && i < d) ? s_head[(size_t)i * d + j] : 0.0f;
        ur[ii] = i < d ? u[head * d + i] : 0.0f;
    }

    auto fetch = [&](int tile0, int buf) {               // the tile's inputs on their way into buffer `buf`
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            const int e = tid + x * THREADS, tt = e / DMAX, c = e % DMAX;
            const bool ok = tile0 + tt < t1 && c < d;
            const size_t at = ok ? (size_t)(tile0 + tt) * in_stride + head * d + c : 0;
            cp_async4(&rs[buf][tt][c], r + at, ok);
            cp_async4(&ks[buf][tt][c], k + at, ok);
            cp_async4(&as[buf][tt][c], a + at, ok);
        }
#pragma unroll
        for (int x = 0; x < PERC; ++x) {
            const int e = tid + x * THREADS, tt = e / DC, c = c0 + e % DC;
            if (e >= WKV_TT * DC) break;
            const bool ok = tile0 + tt < t1 && c < d;
            const size_t at = ok ? (size_t)(tile0 + tt) * in_stride + head * d + c : 0;
            cp_async4(&vs[buf][tt][e % DC], v + at, ok);
            if (JS == 1) cp_async4(&gs[buf][tt][e % DC], g + at, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    if (t0 < t1) fetch(t0, 0);
    int buf = 0;
    for (int tile0 = t0; tile0 < t1; tile0 += WKV_TT, buf ^= 1) {
        // the buffer that is filled next was read two tiles ago; everyone has left that tile
        if (tile0 + WKV_TT < t1) {
            fetch(tile0 + WKV_TT, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();                                 // this tile's inputs are here; the tile before is written out
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            const int e = tid + x * THREADS, tt = e / DMAX, c = e % DMAX;
            ws[tt][c] = c < d ? expf(-expf(as[buf][tt][c] + w0[head * d + c])) : 0.0f;
        }
        __syncthreads();
        const int nt = min(WKV_TT, t1 - tile0);
        // every lane keeps its part of o for each token of the tile; the lanes of a column meet once
        // per tile, sixteen independent exchanges in flight, instead of once per token
        float o_part[WKV_TT];
#pragma unroll
        for (int tt = 0; tt < WKV_TT; ++tt) {
            o_part[tt] = 0.0f;
            if (tt < nt) {
                const float vj = vs[buf][tt][j - c0];
                float o = 0.0f;
                const float4* k4 = reinterpret_cast<const float4*>(&ks[buf][tt][part * 4]);
                const float4* r4 = reinterpret_cast<const float4*>(&rs[buf][tt][part * 4]);
                const float4* w4 = reinterpret_cast<const float4*>(&ws[tt][part * 4]);
#pragma unroll
                for (int q4 = 0; q4 < NI / 4; ++q4) {        // four rows a load
                    const float4 kq = k4[q4 * WKV_IS], rq = r4[q4 * WKV_IS], wq = w4[q4 * WKV_IS];
                    const float kk[4] = {kq.x, kq.y, kq.z, kq.w}, rr[4] = {rq.x, rq.y, rq.z, rq.w};
                    const float ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const int ii = q4 * 4 + x;
                        const float kv = kk[x] * vj;
                        o = fmaf(rr[x], fmaf(ur[ii], kv, S[ii]), o);
                        S[ii] = fmaf(ww[x], S[ii], kv);
                    }
                }
                o_part[tt] = o;
            }
        }
#pragma unroll
        for (int sh = 1; sh < WKV_IS; sh *= 2) {
#pragma unroll
            for (int tt = 0; tt < WKV_TT; ++tt) o_part[tt] += __shfl_xor_sync(0xffffffffu, o_part[tt], sh);
        }
        if (part == 0) {
#pragma unroll
            for (int tt = 0; tt < WKV_TT; ++tt)
                if (tt < nt) os[tt][j - c0] = live ? o_part[tt] : 0.0f;
        }
        __syncthreads();
        if (JS > 1) {                                    // the row's other columns are elsewhere
            for (int e = tid; e < nt * DC; e += THREADS) {
                const int tt = e / DC, c = c0 + e % DC;
                if (c < d) o_raw[(size_t)(tile0 + tt) * num_heads * d + head * d + c] = os[tt][e % DC];
            }
            continue;
        }
        for (int tt = tid / 32; tt < nt; tt += THREADS / 32) {       // a warp per token: its unit norm
            float ss = 0.0f;
            for (int c = tid % 32; c < d; c += 32) ss = fmaf(os[tt][c], os[tt][c], ss);
            ss = warp_sum(ss);
            if (tid % 32 == 0) inv_s[tt] = 1.0f / sqrtf(ss / (float)d + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * DC; e += THREADS) {
            const int tt = e / DC, c = e % DC;
            if (c < d) {
                const float gj = gs[buf][tt][c];
                const float y = os[tt][c] * inv_s[tt] * norm_weight[head * d + c] * (gj / (1.0f + expf(-gj)));
                out[(size_t)(tile0 + tt) * num_heads * d + head * d + c] = from_f32<TO>(y);
            }
        }
    }
    if (t1 > t0) {
        if (live) {
#pragma unroll
            for (int ii = 0; ii < NI; ++ii) {
                const int i = (ii / 4) * (4 * WKV_IS) + part * 4 + ii % 4;
                if (i < d) s_head[(size_t)i * d + j] = S[ii];
            }
        }
        if (head == 0 && blockIdx.z == 0) {
            const TH* last = h + (size_t)(t1 - 1) * width;
            for (int e = tid; e < width; e += THREADS) slot[prev_offset + e] = to_f32(last[e]);
        }
    }
}

// out[t, head] = o / rms(o) * weight * silu(g) for the rows that column-split blocks left as float32:
// a warp per (token, head)
template <typename TO>
__global__ void __launch_bounds__(256)
wkv_finish_kernel(const float* o_raw, const float* g, int g_stride, const float* __restrict__ norm_weight, float eps,
                  int num_items, int num_heads, int d, TO* __restrict__ out) {
    const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= num_items) return;
    const int t = item / num_heads, head = item % num_heads;
    const float* o = o_raw + (size_t)item * d;
    float ss = 0.0f;
    for (int c = lane; c < d; c += 32) ss = fmaf(o[c], o[c], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
    for (int c = lane; c < d; c += 32) {
        const float gj = g[(size_t)t * g_stride + head * d + c];
        out[(size_t)item * d + c] = from_f32<TO>(o[c] * inv * norm_weight[head * d + c] * (gj / (1.0f + expf(-gj))));
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

// col_split: 1, or 4 to cut a head's state columns over four blocks (o_raw: float32 [T, heads * d] scratch)
extern "C" int ti_wkv_recurrence(const float* r, const float* k, const float* v, const float* g, const float* a,
                                 int in_stride, const float* w0, const float* u, const float* norm_weight,
                                 float eps, const void* h, int h_dtype, int width, const int* cu_q,
                                 const int* slots, float* state, long long state_stride, long long prev_offset,
                                 int num_requests, int num_tokens, int num_heads, int d, int col_split,
                                 float* o_raw, void* out, void* stream) {
    if (num_requests == 0) return 0;
    TI_REQUIRE(d >= 1 && d <= 128, "wkv_recurrence: head size %d must be at most 128", d);
    TI_REQUIRE(col_split == 1 || (col_split == 4 && o_raw != nullptr), "wkv_recurrence: columns are cut over 1 or 4 "
               "blocks, and four need scratch");
    dim3 grid(num_requests, num_heads, col_split);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TH, DMAX, JS)                                                                       \
    wkv_recurrence_kernel<TH, TH, DMAX, JS><<<grid, DMAX / JS * wkv_lanes(DMAX, JS), 0, s>>>(                      \
        r, k, v, g, a, in_stride, w0, u, norm_weight, eps, (const TH*)h, width, cu_q, slots, state,    \
        (size_t)state_stride, (size_t)prev_offset, num_heads, d, (TH*)out, o_raw)
#define CALL(TH)                                                                                   \
    if (col_split == 4) {                                                                          \
        if (d <= 32) LAUNCH(TH, 32, 4); else if (d <= 64) LAUNCH(TH, 64, 4); else LAUNCH(TH, 128, 4); \
        if (int rc = ti_check_launch("wkv_recurrence")) return rc;                                 \
        const int items = num_tokens * num_heads;                                                  \
        wkv_finish_kernel<TH><<<(items + 7) / 8, 256, 0, s>>>(o_raw, g, in_stride, norm_weight, eps, items, \
                                                            num_heads, d, (TH*)out);               \
        return ti_check_launch("wkv_finish");                                                      \
    }                                                                                              \
    if (d <= 32) LAUNCH(TH, 32, 1); else if (d <= 64) LAUNCH(TH, 64, 1); else LAUNCH(TH, 128, 1)
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
