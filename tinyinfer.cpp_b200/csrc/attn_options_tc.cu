// Paged flash attention with optional parts on the tensor cores (bfloat16 operands, mma.sync
// m16n8k16), for prompt portions and single decoded tokens alike.
//
// The options are those of attention_options (attn_options.cu): a window and/or chunks of
// positions, a score factor per head, a cap on the score, a sink in the softmax, an output gate
// per head or per element, and pages that hold one shared row per token (key = the row, value =
// its first dv elements).
//
// Arrangement.  A block has 64 rows (4 warps x 16).  A row is a (token, query head) pair: the
// heads of one kv group (padded to a power of two, GP) of 64 / GP consecutive tokens of one
// request, so a tile of keys and values is fetched once for all heads that read it (one shared
// row serves every head of a latent layer).  The block walks its keys in tiles of 64 through a
// two-stage cp.async ring, from the first key any of its rows may see to its last row's own
// position; masks are applied only in tiles that touch an edge.  Queries lie in shared memory
// (a row of queries may be wide: a latent row), the head size is a runtime multiple of 16.
// A block makes DVS of the value columns; wider values are cut into slices, a block each.
// Few rows (decoding) cut the keys of a row into runs of tiles, a block each, whose unnormalised
// results a second launch adds (attn_options_merge); and when a tile has at most 16 rows (single
// tokens, up to 16 heads per kv head) the four warps of a block share those rows and take a
// quarter of every tile's keys each, meeting in shared memory at the end.
//
// Precision.  Scores, cap (with the hardware's float32 exponential and reciprocal, relative error
// about 2^-22), softmax weights and sums are float32.  The weighted sum of the values
// also takes the weights in full float32: a weight is split into three bfloat16 parts (8 + 8 + 8
// bits of its significand), each multiplies the bfloat16 values on the tensor cores, and the
// three products are added in the float32 accumulator.
#include "common.cuh"

namespace {

constexpr int BM = 64;
constexpr int BN = 64;
constexpr int STAGES = 2;
constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two floats as three pairs of bfloat16 whose sums are the floats: the upper 16 bits of a float
// are a bfloat16 (truncated), what is left is exact in float32 and is cut the same way again;
// after three cuts nothing of the 24-bit significand is left.
__device__ __forceinline__ void split3_pair(float x, float y, unsigned& hi, unsigned& mid, unsigned& lo) {
    const unsigned xb = __float_as_uint(x), yb = __float_as_uint(y);
    hi = __byte_perm(xb, yb, 0x7632);
    const float x1 = x - __uint_as_float(xb & 0xffff0000u), y1 = y - __uint_as_float(yb & 0xffff0000u);
    const unsigned x1b = __float_as_uint(x1), y1b = __float_as_uint(y1);
    mid = __byte_perm(x1b, y1b, 0x7632);
    const float x2 = x1 - __uint_as_float(x1b & 0xffff0000u), y2 = y1 - __uint_as_float(y1b & 0xffff0000u);
    lo = __byte_perm(__float_as_uint(x2), __float_as_uint(y2), 0x7632);
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct TcOptions {
    int window, chunk;
    float scale, softcap;
    const float* head_scale;
    const float* sink;
    const float* gate;
    int gate_stride, gate_per_head, shared_rows;
};

__device__ __forceinline__ int first_visible(int p, const TcOptions& o) {
    int lo = o.window > 0 ? max(0, p - o.window + 1) : 0;
    if (o.chunk > 0) lo = max(lo, p / o.chunk * o.chunk);
    return lo;
}

// tiles[i] = {request row, first flat token, tokens (<= 64 / gp)}
// MODE 0: the warps of a block have 16 rows each.  MODE 1 (KS): all have the same 16 rows and a quarter
// of a tile's keys.  MODE 2 (shared rows, at most 16 live rows, up to four slices of value columns):
// all have the same 16 rows and all keys, and warp w makes slice w of the value columns, so that a
// tile of rows is fetched once for all of them.
template <int DVS, int MODE>
__global__ void __launch_bounds__(WARPS * 32)
attn_options_tc_kernel(const bf16* q, const int* __restrict__ tiles, const int* __restrict__ positions,
                       const int* __restrict__ block_table, int bt_stride, const bf16* pages, int num_pages,
                       int page_size, int num_heads, int num_kv_heads, int dk, int dv, int gp, int head_blocks,
                       int nsplit, TcOptions opt, bf16* __restrict__ out, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int* __restrict__ status) {
    constexpr int NT_O = DVS / 8;
    constexpr bool KS = MODE == 1;
    constexpr int V_ROW = DVS * 2 + 16;
    // KS (at most 16 live rows, decoding): every warp has the same 16 rows and a quarter of a tile's keys
    constexpr int NJ = KS ? BN / 32 : BN / 8;            // 8-key columns of a tile that a warp multiplies
    extern __shared__ __align__(16) unsigned char smem[];
    const int k_row = dk * 2 + 16;                       // bytes of a staged query or key row
    const int stage_bytes = BN * k_row + (opt.shared_rows ? 0 : BN * V_ROW);
    unsigned char* q_s = smem;
    unsigned char* ring = smem + BM * k_row;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int rbase = MODE == 0 ? warp * 16 : 0, kbase = KS ? warp * 16 : 0;
    const int slices = MODE == 2 ? 1 : dv / DVS;         // slices that the grid spreads over blocks
    int bx = blockIdx.x;
    const int slice = MODE == 2 ? warp : bx % slices; bx /= slices;
    const int hb = bx % head_blocks; const int kvh = bx / head_blocks;
    const int group = num_heads / num_kv_heads;
    const int tile_id = blockIdx.y, split = blockIdx.z;
    const int req = tiles[tile_id * 3], tok0 = tiles[tile_id * 3 + 1], ntok = tiles[tile_id * 3 + 2];
    const int* table = block_table + (size_t)req * bt_stride;
    const size_t page_elems = (size_t)num_kv_heads * page_size * (opt.shared_rows ? dk : dk + dv);
    const size_t v_base = (size_t)num_kv_heads * page_size * dk;

    const int pos_first = positions[tok0], pos_last = pos_first + ntok - 1;
    const int kv_lo = first_visible(pos_first, opt);
    int kt_lo = kv_lo / BN, kt_hi = pos_last / BN + 1;
    if (nsplit > 1) {                                    // this block's run of the key tiles
        const int per = (kt_hi - kt_lo + nsplit - 1) / nsplit;
        kt_lo += split * per;
        kt_hi = min(kt_hi, kt_lo + per);
    }

    // row i of the block: token i / gp, head hb * gp + i % gp of the kv group
    auto row_token = [&](int i) { return i / gp; };
    auto row_head = [&](int i) {
        const int hg = hb * gp + i % gp;
        return (i / gp < ntok && hg < group) ? kvh * group + hg : -1;
    };
    int row_pos[2], row_lo[2], row_h[2];
    float row_scale[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = rbase + g + 8 * r;
        row_h[r] = row_head(i);
        row_pos[r] = row_h[r] >= 0 ? pos_first + row_token(i) : -1;
        row_lo[r] = row_h[r] >= 0 ? first_visible(row_pos[r], opt) : 0;
        row_scale[r] = opt.scale * ((opt.head_scale && row_h[r] >= 0) ? opt.head_scale[row_h[r]] : 1.0f);
    }
    const float cap_arg = opt.softcap > 0.0f ? 2.0f * LOG2E / opt.softcap : 0.0f, cap_l2e = opt.softcap * LOG2E;
    const int warp_tok_lo = min(ntok - 1, rbase / gp), warp_tok_hi = min(ntok - 1, (rbase + 15) / gp);
    const bool warp_live = rbase / gp < ntok && (MODE != 2 || warp < dv / DVS);
    const int warp_pos_lo = pos_first + warp_tok_lo, warp_pos_hi = pos_first + warp_tok_hi;
    const int warp_lo_first = first_visible(warp_pos_lo, opt), warp_lo_last = first_visible(warp_pos_hi, opt);

    // queries into shared memory (part of the first commit group)
    const int chunks = dk / 8;
    for (int c = threadIdx.x; c < BM * chunks; c += WARPS * 32) {
        const int i = c / chunks, part = c % chunks;
        const int h = row_head(i);
        const bf16* src = h >= 0 ? q + ((size_t)(tok0 + row_token(i)) * num_heads + h) * dk + part * 8 : q;
        cp_async16(q_s + (size_t)i * k_row + part * 16, src, h >= 0);
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    auto issue = [&](int kt, int stage) {
        unsigned char* kdst = ring + (size_t)stage * stage_bytes;
        unsigned char* vdst = kdst + BN * k_row;
#pragma unroll
        for (int r = 0; r < BN / 16; ++r) {              // four runs of 16 keys, each inside one page
            const int key0 = kt * BN + r * 16;
            int pg = -1;
            if (key0 <= pos_last && key0 + 16 > kv_lo) {
                pg = table[key0 / page_size];
                if (pg < 0 || pg >= num_pages) {
                    if (threadIdx.x == 0) atomicCAS(status, 0, 1);
                    pg = -1;
                }
            }
            const bool valid = pg >= 0;
            const bf16* base = pages + (valid ? (size_t)pg * page_elems : 0);
            const bf16* ksrc = base + (valid ? ((size_t)kvh * page_size + key0 % page_size) * dk : 0);
            for (int c = threadIdx.x; c < 16 * chunks; c += WARPS * 32)
                cp_async16(kdst + (size_t)(r * 16 + c / chunks) * k_row + (c % chunks) * 16,
                           ksrc + (valid ? c * 8 : 0), valid);
            if (!opt.shared_rows) {
                const bf16* vsrc = base + (valid ? v_base + ((size_t)kvh * page_size + key0 % page_size) * dv
                                                       + slice * DVS : 0);
                constexpr int VCH = DVS / 8;
                for (int c = threadIdx.x; c < 16 * VCH; c += WARPS * 32)
                    cp_async16(vdst + (size_t)(r * 16 + c / VCH) * V_ROW + (c % VCH) * 16,
                               vsrc + (valid ? (size_t)(c / VCH) * dv + (c % VCH) * 8 : 0), valid);
            }
        }
    };

    if (kt_lo < kt_hi) issue(kt_lo, 0);
    cp_async_commit();
    const int ksteps = dk / 16;
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int stage = (kt - kt_lo) % STAGES;
        if (kt + 1 < kt_hi) issue(kt + 1, (kt + 1 - kt_lo) % STAGES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key_lo = kt * BN + kbase, key_hi = key_lo + NJ * 8 - 1;     // the warp's keys of the tile
        const bool visible = warp_live && key_lo <= warp_pos_hi && key_hi >= warp_lo_first;
        if (visible) {
            const unsigned char* ks = ring + (size_t)stage * stage_bytes;
            const unsigned char* vs = opt.shared_rows ? ks + (size_t)slice * DVS * 2 : ks + BN * k_row;
            const int v_row = opt.shared_rows ? k_row : V_ROW;
            float s_acc[NJ][4];
#pragma unroll
            for (int j = 0; j < NJ; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
            for (int kk = 0; kk < ksteps; ++kk) {
                unsigned qa[4];
                ldmatrix_x4(qa, q_s + (size_t)(rbase + (lane & 7) + ((lane >> 3) & 1) * 8) * k_row
                                    + (kk * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
                for (int jp = 0; jp < NJ / 2; ++jp) {
                    unsigned b[4];
                    const int key = kbase + jp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + (size_t)key * k_row + dim * 2);
                    mma_bf16(s_acc[2 * jp], qa, b[0], b[1]);
                    mma_bf16(s_acc[2 * jp + 1], qa, b[2], b[3]);
                }
            }
            const bool edge = key_hi > warp_pos_lo || key_lo < warp_lo_last;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s_acc[j][e] * row_scale[e >> 1];
                    if (opt.softcap > 0.0f)      // cap tanh(v / cap) = cap (1 - 2 / (exp(2 v / cap) + 1))
                        v = cap_l2e * fmaf(-2.0f, rcp_approx(ex2_approx(v * cap_arg) + 1.0f), 1.0f);
                    else
                        v *= LOG2E;
                    if (edge) {
                        const int key = key_lo + j * 8 + tq * 2 + (e & 1);
                        if (key > row_pos[e >> 1] || key < row_lo[e >> 1]) v = -INFINITY;
                    }
                    s_acc[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float alpha[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = m_new == -INFINITY ? 1.0f : exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
                m_use[r] = m_new == -INFINITY ? 0.0f : m_new;     // a row that sees nothing yet
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(s_acc[j][e] - m_use[e >> 1]);
                    s_acc[j][e] = p;
                    sum[e >> 1] += p;
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + sum[r];
            if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
                for (int i = 0; i < NT_O; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < NJ / 2; ++kk) {
                unsigned pa[3][4];
#pragma unroll
                for (int x = 0; x < 4; ++x)               // fragment register x: tile 2kk + (x >> 1), elements (x & 1) * 2, +1
                    split3_pair(s_acc[2 * kk + (x >> 1)][(x & 1) * 2], s_acc[2 * kk + (x >> 1)][(x & 1) * 2 + 1],
                                pa[0][x], pa[1][x], pa[2][x]);
                // value fragments of up to four column pairs at a time, so that the products into one
                // accumulator stand eight apart
                constexpr int DPG = NT_O / 2 < 4 ? NT_O / 2 : 4;
#pragma unroll
                for (int dp0 = 0; dp0 < NT_O / 2; dp0 += DPG) {
                    unsigned b[DPG][4];
                    const int key = kbase + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int x = 0; x < DPG; ++x)
                        ldmatrix_x4_trans(b[x], vs + (size_t)key * v_row + ((dp0 + x) * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
                    for (int part = 2; part >= 0; --part) {       // the smallest parts first
#pragma unroll
                        for (int x = 0; x < DPG; ++x) {
                            mma_bf16(o[2 * (dp0 + x)], pa[part], b[x][0], b[x][1]);
                            mma_bf16(o[2 * (dp0 + x) + 1], pa[part], b[x][2], b[x][3]);
                        }
                    }
                }
            }
        }
        __syncthreads();                              // the stage may be refilled
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (KS) {
        // the four warps hold the same rows over different keys: their maxima, sums and outputs
        // meet in shared memory (the ring is free now), and every thread finishes some elements
        float* m_s = reinterpret_cast<float*>(ring);          // [4][16]
        float* l_s = m_s + WARPS * 16;                        // [4][16]
        float* o_s = l_s + WARPS * 16;                        // [4][16][DVS]
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            if (tq == 0) { m_s[warp * 16 + row] = m_run[r]; l_s[warp * 16 + row] = l_run[r]; }
#pragma unroll
            for (int x = 0; x < NT_O; ++x) {
                o_s[(warp * 16 + row) * DVS + x * 8 + tq * 2] = o[x][2 * r];
                o_s[(warp * 16 + row) * DVS + x * 8 + tq * 2 + 1] = o[x][2 * r + 1];
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 16 * DVS; e += WARPS * 32) {
            const int row = e / DVS, col = e % DVS;
            const int h = row_head(row);
            if (h < 0) continue;
            const int t = tok0 + row_token(row);
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) m = fmaxf(m, m_s[w * 16 + row]);
            float l = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = m_s[w * 16 + row];
                const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
                l = fmaf(l_s[w * 16 + row], f, l);
                acc = fmaf(o_s[(w * 16 + row) * DVS + col], f, acc);
            }
            if (nsplit > 1) {
                const size_t at = ((size_t)t * num_heads + h) * nsplit + split;
                part_o[at * dv + slice * DVS + col] = acc;
                if (col == 0 && slice == 0) { part_ml[at * 2] = m; part_ml[at * 2 + 1] = l; }
                continue;
            }
            if (opt.sink) l += exp2f(opt.sink[h] * LOG2E - m);
            acc /= l;
            if (opt.gate) {
                const float* gt = opt.gate + (size_t)t * opt.gate_stride;
                const float gv = opt.gate_per_head ? gt[h] : gt[(size_t)h * dv + slice * DVS + col];
                acc *= 1.0f / (1.0f + expf(-gv));
            }
            out[((size_t)t * num_heads + h) * dv + slice * DVS + col] = __float2bfloat16_rn(acc);
        }
        return;
    }
    if (MODE == 2 && slice >= dv / DVS) return;      // a warp without a slice of its own has nothing to write
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int h = row_h[r];
        if (h < 0) continue;
        const int t = tok0 + row_token(rbase + g + 8 * r);
        if (nsplit > 1) {                             // unnormalised, for the merging launch
            const size_t at = ((size_t)t * num_heads + h) * nsplit + split;
            float* po = part_o + at * dv + slice * DVS + tq * 2;
#pragma unroll
            for (int x = 0; x < NT_O; ++x) {
                po[x * 8] = o[x][2 * r];
                po[x * 8 + 1] = o[x][2 * r + 1];
            }
            if (tq == 0 && slice == 0) { part_ml[at * 2] = m_run[r]; part_ml[at * 2 + 1] = l_run[r]; }
            continue;
        }
        float l = l_run[r];
        if (opt.sink) l += exp2f(opt.sink[h] * LOG2E - m_run[r]);
        float inv = 1.0f / l;
        const float* gt = opt.gate ? opt.gate + (size_t)t * opt.gate_stride : nullptr;
        if (gt && opt.gate_per_head) inv *= 1.0f / (1.0f + expf(-gt[h]));
        bf16* op = out + ((size_t)t * num_heads + h) * dv + slice * DVS + tq * 2;
        const float* ge = (gt && !opt.gate_per_head) ? gt + (size_t)h * dv + slice * DVS + tq * 2 : nullptr;
#pragma unroll
        for (int x = 0; x < NT_O; ++x) {
            float a = o[x][2 * r] * inv, b = o[x][2 * r + 1] * inv;
            if (ge) { a *= 1.0f / (1.0f + expf(-ge[x * 8])); b *= 1.0f / (1.0f + expf(-ge[x * 8 + 1])); }
            *reinterpret_cast<__nv_bfloat162*>(op + x * 8) = __floats2bfloat162_rn(a, b);
        }
    }
}

// adds the runs of a row's keys: blocks of 128 value columns of a (token, head); the runs' factors are made once,
// and a thread has several loads in flight
__global__ void __launch_bounds__(128)
attn_options_merge_kernel(const float* part_o, const float* part_ml, int nsplit, int num_heads, int dv,
                          const float* __restrict__ sink, const float* gate, int gate_stride, int gate_per_head,
                          bf16* __restrict__ out) {
    __shared__ float f_s[64];
    __shared__ float inv_s;
    const int item = blockIdx.x, t = item / num_heads, h = item % num_heads;
    const float* ml = part_ml + (size_t)item * nsplit * 2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float m0 = lane < nsplit ? ml[lane * 2] : -INFINITY, m1 = lane + 32 < nsplit ? ml[(lane + 32) * 2] : -INFINITY;
        const float m = warp_max(fmaxf(m0, m1));
        const float f0 = m0 == -INFINITY ? 0.0f : exp2f(m0 - m), f1 = m1 == -INFINITY ? 0.0f : exp2f(m1 - m);
        float l = (lane < nsplit ? ml[lane * 2 + 1] * f0 : 0.0f) + (lane + 32 < nsplit ? ml[(lane + 32) * 2 + 1] * f1 : 0.0f);
        l = warp_sum(l);
        if (sink) l += exp2f(sink[h] * LOG2E - m);
        f_s[lane] = f0; f_s[lane + 32] = f1;
        if (lane == 0) {
            float inv = 1.0f / l;
            if (gate && gate_per_head) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
            inv_s = inv;
        }
    }
    __syncthreads();
    const float* po = part_o + (size_t)item * nsplit * dv;
    for (int d = blockIdx.y * 128 + threadIdx.x; d < dv; d += 128 * gridDim.y) {
        float acc = 0.0f;
#pragma unroll 8
        for (int z = 0; z < nsplit; ++z) acc = fmaf(po[(size_t)z * dv + d], f_s[z], acc);
        acc *= inv_s;
        if (gate && !gate_per_head) acc *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + (size_t)h * dv + d]));
        out[(size_t)item * dv + d] = __float2bfloat16_rn(acc);
    }
}

// out[t, h, :] = x[t, h, :] W[h] on the tensor cores, for many tokens: a block has 64 tokens of one head and
// 128 columns; the tokens' rows lie in shared memory, W[h] ([n_in, n_out], columns contiguous) comes in runs
// of 64 of its rows through a two-stage cp.async ring and is read transposed, as the values of the attention
// kernel are.
constexpr int HPK = 64;          // rows of W[h] a stage holds
constexpr int HP_WROW = 128 * 2 + 16;

__global__ void __launch_bounds__(WARPS * 32)
head_project_tc_kernel(const bf16* x, int x_stride_t, int x_stride_h, const bf16* __restrict__ w, int n_in, int n_out,
                       bf16* out, int out_stride_t, int out_stride_h, int num_tokens) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int x_row = n_in * 2 + 16;
    unsigned char* xs = smem;
    unsigned char* ring = smem + (size_t)BM * x_row;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int t0 = blockIdx.x * BM, h = blockIdx.y, n0 = blockIdx.z * 128;
    const int chunks = n_in / 8;
    for (int c = threadIdx.x; c < BM * chunks; c += WARPS * 32) {
        const int i = c / chunks, part = c % chunks;
        const bool ok = t0 + i < num_tokens;
        cp_async16(xs + (size_t)i * x_row + part * 16,
                   x + (ok ? (size_t)(t0 + i) * x_stride_t + (size_t)h * x_stride_h + part * 8 : 0), ok);
    }
    const bf16* wh = w + (size_t)h * n_in * n_out;
    auto issue = [&](int kc, int stage) {
        unsigned char* dst = ring + (size_t)stage * HPK * HP_WROW;
        for (int c = threadIdx.x; c < HPK * 16; c += WARPS * 32) {
            const int k = kc * HPK + c / 16, col = n0 + (c % 16) * 8;
            const bool ok = k < n_in && col < n_out;
            cp_async16(dst + (size_t)(c / 16) * HP_WROW + (c % 16) * 16, wh + (ok ? (size_t)k * n_out + col : 0), ok);
        }
    };
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const int num_kc = (n_in + HPK - 1) / HPK;
    issue(0, 0);
    cp_async_commit();
    for (int kc = 0; kc < num_kc; ++kc) {
        if (kc + 1 < num_kc) issue(kc + 1, (kc + 1) % STAGES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* ws = ring + (size_t)(kc % STAGES) * HPK * HP_WROW;
        const int steps = min(HPK, n_in - kc * HPK) / 16;
        for (int ks = 0; ks < steps; ++ks) {
            unsigned a[4];
            ldmatrix_x4(a, xs + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * x_row
                               + (kc * HPK + ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                unsigned b[4];
                const int k = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                ldmatrix_x4_trans(b, ws + (size_t)k * HP_WROW + (dp * 16 + (lane >> 4) * 8) * 2);
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int t = t0 + warp * 16 + g + 8 * r;
        if (t >= num_tokens) continue;
        bf16* dst = out + (size_t)t * out_stride_t + (size_t)h * out_stride_h + n0 + tq * 2;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int col = n0 + i * 8 + tq * 2;
            if (col < n_out) dst[i * 8] = __float2bfloat16_rn(o[i][2 * r]);
            if (col + 1 < n_out) dst[i * 8 + 1] = __float2bfloat16_rn(o[i][2 * r + 1]);
        }
    }
}

int value_slice(int dv) { return dv % 128 == 0 ? 128 : dv % 64 == 0 ? 64 : dv % 32 == 0 ? 32 : 16; }

size_t smem_bytes(int dk, int dv, int shared_rows) {
    const size_t k_row = (size_t)dk * 2 + 16, v_row = (size_t)value_slice(dv) * 2 + 16;
    const size_t ring = STAGES * (BN * k_row + (shared_rows ? 0 : BN * v_row));
    const size_t meet = (size_t)WARPS * 16 * (value_slice(dv) + 2) * sizeof(float);     // where split warps meet
    return BM * k_row + (ring > meet ? ring : meet);
}

}  // namespace

extern "C" int ti_attn_options_tc_supported(int dk, int dv, int page_size, int shared_rows) {
    return dk >= 16 && dk % 16 == 0 && dv >= 16 && dv % 16 == 0 && page_size >= 16 && page_size % 16 == 0 &&
           (!shared_rows || dv <= dk) && smem_bytes(dk, dv, shared_rows) <= 227 * 1024;
}

extern "C" int ti_head_project_tc_supported(int n_in, int n_out, int x_stride_t, int x_stride_h) {
    return n_in >= 16 && n_in % 16 == 0 && n_out % 8 == 0 && x_stride_t % 8 == 0 && x_stride_h % 8 == 0 &&
           (size_t)BM * (n_in * 2 + 16) + (size_t)STAGES * HPK * HP_WROW <= 227 * 1024;
}

// x: bfloat16 [T, heads, n_in] (strides over tokens and heads, 16-byte aligned rows), w: bfloat16 [heads, n_in, n_out],
// out: bfloat16 [T, heads, n_out] (strides over tokens and heads)
extern "C" int ti_head_project_tc(const void* x, int x_stride_t, int x_stride_h, const void* w, int n_in, int n_out,
                                  void* out, int out_stride_t, int out_stride_h, int num_tokens, int num_heads,
                                  void* stream) {
    if (num_tokens == 0 || num_heads == 0) return 0;
    TI_REQUIRE(ti_head_project_tc_supported(n_in, n_out, x_stride_t, x_stride_h) && (uintptr_t)x % 16 == 0 &&
               (uintptr_t)w % 16 == 0, "head_project_tc: sizes %d x %d, strides %d, %d or alignment are not supported",
               n_in, n_out, x_stride_t, x_stride_h);
    const size_t smem = (size_t)BM * (n_in * 2 + 16) + (size_t)STAGES * HPK * HP_WROW;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(head_project_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) return ti_fail("head_project_tc: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid((num_tokens + BM - 1) / BM, num_heads, (n_out + 127) / 128);
    head_project_tc_kernel<<<grid, WARPS * 32, smem, (cudaStream_t)stream>>>(
        (const bf16*)x, x_stride_t, x_stride_h, (const bf16*)w, n_in, n_out, (bf16*)out, out_stride_t, out_stride_h,
        num_tokens);
    return ti_check_launch("head_project_tc");
}

// rows of a block that belong to one token: the heads of a kv group, padded to a power of two (at most 64)
extern "C" int ti_attn_options_tc_group_rows(int num_heads, int num_kv_heads) {
    const int group = num_heads / num_kv_heads;
    int gp = 1;
    while (gp < group && gp < BM) gp *= 2;
    return gp;
}

// tiles: int32 [num_tiles, 3] = {request row, first flat token, tokens}; a tile has at most
// 64 / group_rows consecutive tokens of one request.  part_o/part_ml: float32 scratch of
// [tokens, heads, nsplit, dv] and [tokens, heads, nsplit, 2] when nsplit > 1.  key_split: every tile has at
// most 16 rows (tokens x group_rows), and the warps of a block share them and split a tile's keys (1) or,
// with shared rows, the slices of the value columns (2; every tile is then a single token, and a group of more
// than 16 heads is spread over blocks of 16).
extern "C" int ti_attn_options_tc(const void* q, const int* tiles, int num_tiles, int num_tokens,
                                  const int* positions, const int* block_table, int bt_stride, const void* pages,
                                  int num_pages, int page_size, int num_heads, int num_kv_heads, int dk, int dv,
                                  int shared_rows, int window, int chunk, float scale, float softcap,
                                  const float* head_scale, const float* sink, const float* gate, int gate_stride,
                                  int gate_per_head, int nsplit, float* part_o, float* part_ml, int key_split,
                                  void* out, int* status, void* stream) {
    if (num_tiles == 0) return 0;
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attn_options_tc: %d heads over %d kv heads", num_heads, num_kv_heads);
    TI_REQUIRE(ti_attn_options_tc_supported(dk, dv, page_size, shared_rows),
               "attn_options_tc: head sizes %d and %d (multiples of 16 that fit into shared memory) or page size %d "
               "(a multiple of 16) are not supported", dk, dv, page_size);
    TI_REQUIRE(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || (part_o && part_ml)), "attn_options_tc: runs and scratch");
    TI_REQUIRE(num_tiles <= 65535, "attn_options_tc: %d tiles exceed the grid limit", num_tiles);
    TI_REQUIRE(key_split != 1 || ti_attn_options_tc_group_rows(num_heads, num_kv_heads) <= 16,
               "attn_options_tc: warps split the keys only when a tile has at most 16 rows");
    int gp = ti_attn_options_tc_group_rows(num_heads, num_kv_heads);
    if (key_split == 2 && gp > 16) gp = 16;      // a tile is one token: more heads than 16 take several blocks
    const int group = num_heads / num_kv_heads, head_blocks = (group + gp - 1) / gp;
    // prompt portions over shared rows: 256 value columns a block where they divide, so that the score
    // product of a wide row is repeated half as often (such a block fills an SM's shared memory anyway)
    const int dvs = (shared_rows && key_split == 0 && dv % 256 == 0) ? 256 : value_slice(dv);
    const size_t smem = smem_bytes(dk, dv, shared_rows);
    TcOptions opt = {window, chunk, scale, softcap, head_scale, sink, gate, gate_stride, gate_per_head, shared_rows};
    TI_REQUIRE(key_split != 2 || (shared_rows && dv / dvs <= WARPS), "attn_options_tc: a warp per slice needs shared rows "
               "and at most %d slices", WARPS);
    dim3 grid(num_kv_heads * head_blocks * (key_split == 2 ? 1 : dv / dvs), num_tiles, nsplit);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(DVS, MODE)                                                                                       \
    {                                                                                                     \
        static TiPerDevice configured;                                                                    \
        static size_t allowed = 0;                                                                        \
        if (configured.first_use() || smem > allowed) {                                                   \
            cudaError_t e = cudaFuncSetAttribute(attn_options_tc_kernel<DVS, MODE>,                             \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); \
            if (e != cudaSuccess) return ti_fail("attn_options_tc: %s", cudaGetErrorString(e));           \
            configured.mark();                                                                            \
            allowed = 227 * 1024;                                                                         \
        }                                                                                                 \
        attn_options_tc_kernel<DVS, MODE><<<grid, WARPS * 32, smem, s>>>(                                        \
            (const bf16*)q, tiles, positions, block_table, bt_stride, (const bf16*)pages, num_pages,       \
            page_size, num_heads, num_kv_heads, dk, dv, gp, head_blocks, nsplit, opt, (bf16*)out, part_o,   \
            part_ml, status);                                                                             \
    }
    switch (dvs) {
        case 256: LAUNCH(256, 0) break;
        case 128: if (key_split == 2) LAUNCH(128, 2) else if (key_split) LAUNCH(128, 1) else LAUNCH(128, 0) break;
        case 64: if (key_split == 2) LAUNCH(64, 2) else if (key_split) LAUNCH(64, 1) else LAUNCH(64, 0) break;
        case 32: if (key_split == 2) LAUNCH(32, 2) else if (key_split) LAUNCH(32, 1) else LAUNCH(32, 0) break;
        default: if (key_split == 2) LAUNCH(16, 2) else if (key_split) LAUNCH(16, 1) else LAUNCH(16, 0) break;
    }
#undef LAUNCH
    if (int rc = ti_check_launch("attn_options_tc")) return rc;
    if (nsplit > 1) {
        const int items = num_tokens * num_heads;
        attn_options_merge_kernel<<<dim3(items, (dv + 127) / 128), 128, 0, s>>>(part_o, part_ml, nsplit, num_heads, dv, sink, gate, gate_stride,
                                                       gate_per_head, (bf16*)out);
        return ti_check_launch("attn_options_merge");
    }
    return 0;
}
