// Paged flash attention for prompt portions with a bias per (head, distance), a window that
// keeps a request's first tokens, and an output gate (bfloat16, head_dim a multiple of 16 up to
// 128, values of the keys' head size).
//
// The arrangement is that of attn_prefill.cu: a block takes 64 consecutive query tokens of one
// request and one query head (4 warps x 16 rows) and walks the request's keys in tiles of 64
// through a two-stage cp.async ring; scores and the product with the values run on the tensor
// cores (mma.sync m16n8k16), the softmax is online and float32.  What differs:
//  * the walk starts with the tiles that hold the kept first tokens when the window has left
//    them behind, then goes from the window's edge to the last row's own position;
//  * key j is masked for row i when j > i, or when i - j >= window and j >= keep_first;
//  * the score is (q . k) * scale + bias[head][min(i - j, n_dist - 1)]: the 127 distances a tile
//    can hold are brought into shared memory with the tile;
//  * the normalised output is multiplied by sigmoid(gate) before it is stored.
#include "common.cuh"

namespace {

constexpr int BM = 64;         // query rows per block (must match the host's tile list)
constexpr int BN = 64;         // keys per tile
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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// tiles[i] = {request row, first flat token, number of query rows (<= 64)}
template <int HD>
__global__ void __launch_bounds__(WARPS * 32, HD > 64 ? 3 : 4)
attn_bias_prefill_kernel(const bf16* __restrict__ q, const int* __restrict__ tiles,
                    const int* __restrict__ positions, const int* __restrict__ block_table,
                    int bt_stride, const bf16* __restrict__ pages, int num_pages, int page_size,
                    int num_heads, int num_kv_heads, int window, int keep_first, float scale,
                    const float* __restrict__ dist_bias, int n_dist, const float* gate,
                    int gate_stride, bf16* __restrict__ out, int* __restrict__ status) {
    constexpr int ROW_BYTES = HD * 2 + 16;
    constexpr int CHUNKS = HD / 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    constexpr int STAGE_BYTES = 2 * BN * ROW_BYTES;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float sbias[STAGES][2 * BN];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    // heads run fastest in the grid, tiles are sorted by length: blocks start longest first
    const int h = blockIdx.x, tile_id = blockIdx.y;
    const int kvh = h / (num_heads / num_kv_heads);
    const int req = tiles[tile_id * 3], tok0 = tiles[tile_id * 3 + 1];
    const int nrows = tiles[tile_id * 3 + 2];
    const int* table = block_table + (size_t)req * bt_stride;
    const size_t kv_stride = (size_t)num_kv_heads * page_size * HD;

    const int pos_first = positions[tok0], pos_last = pos_first + nrows - 1;
    const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kt_lo = kv_lo / BN, kt_hi = pos_last / BN + 1;
    // tiles of kept first tokens that the window of the first row has left behind come first
    const int n_pre = min(kt_lo, (keep_first + BN - 1) / BN);
    const int n_walk = n_pre + (kt_hi - kt_lo);
    auto tile_of = [&](int i) { return i < n_pre ? i : kt_lo + (i - n_pre); };
    const float* bias_h = dist_bias + (size_t)h * n_dist;

    // this thread's two rows: warp * 16 + g and + 8; a row past the tile sees nothing
    int row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = warp * 16 + g + 8 * r;
        row_pos[r] = i < nrows ? pos_first + i : -1;
    }
    const int warp_pos_lo = pos_first + warp * 16;                       // first row of the warp
    const int warp_pos_hi = min(pos_last, pos_first + warp * 16 + 15);   // its last real row

    unsigned qa[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int k0 = ks * 16 + tq * 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = warp * 16 + g + 8 * r;
            const bf16* qp = q + ((size_t)(tok0 + i) * num_heads + h) * HD + k0;
            qa[ks][r] = i < nrows ? *reinterpret_cast<const unsigned*>(qp) : 0u;
            qa[ks][r + 2] = i < nrows ? *reinterpret_cast<const unsigned*>(qp + 8) : 0u;
        }
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    auto issue = [&](int kt, int stage) {
        unsigned char* kdst = smem + (size_t)stage * STAGE_BYTES;
        unsigned char* vdst = kdst + BN * ROW_BYTES;
        // four runs of 16 keys; a run is contiguous inside its page
#pragma unroll
        for (int r = 0; r < BN / 16; ++r) {
            const int key0 = kt * BN + r * 16;
            int pg = -1;
            if (key0 <= pos_last && (key0 + 16 > kv_lo || key0 < keep_first)) {
                pg = table[key0 / page_size];
                if (pg < 0 || pg >= num_pages) {
                    if (threadIdx.x == 0) atomicCAS(status, 0, 1);
                    pg = -1;
                }
            }
            const bool valid = pg >= 0;
            const bf16* ksrc = pages;
            if (valid)
                ksrc = pages + (((size_t)pg * 2 * num_kv_heads + kvh) * page_size + key0 % page_size) * HD;
            const bf16* vsrc = valid ? ksrc + kv_stride : pages;
            for (int c = threadIdx.x; c < 16 * CHUNKS; c += WARPS * 32) {
                const int off = (r * 16 + c / CHUNKS) * ROW_BYTES + (c % CHUNKS) * 16;
                cp_async16(kdst + off, ksrc + (valid ? c * 8 : 0), valid);
                cp_async16(vdst + off, vsrc + (valid ? c * 8 : 0), valid);
            }
        }
        // the bias of every distance between a row of the block and a key of the tile:
        // entry d stands for distance (pos_first - key_hi) + d
        {
            const int d = pos_first - (kt * BN + BN - 1) + (int)threadIdx.x;
            sbias[stage][threadIdx.x] = bias_h[min(max(d, 0), n_dist - 1)];
        }
    };

    issue(tile_of(0), 0);
    cp_async_commit();
    for (int wi = 0; wi < n_walk; ++wi) {
        const int kt = tile_of(wi);
        const int stage = wi % STAGES;
        if (wi + 1 < n_walk) issue(tile_of(wi + 1), (wi + 1) % STAGES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key_lo = kt * BN, key_hi = key_lo + BN - 1;
        // the warp skips tiles none of its rows can see
        const bool visible = key_lo <= warp_pos_hi &&
                             (window <= 0 || key_hi > warp_pos_lo - window || key_lo < keep_first);
        if (visible) {
            const unsigned char* ks = smem + (size_t)stage * STAGE_BYTES;
            const unsigned char* vs = ks + BN * ROW_BYTES;
            float s_acc[BN / 8][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < BN / 16; ++jp) {
                    unsigned b[4];
                    const int key = jp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + key * ROW_BYTES + dim * 2);
                    mma_bf16(s_acc[2 * jp], qa[kk], b[0], b[1]);
                    mma_bf16(s_acc[2 * jp + 1], qa[kk], b[2], b[3]);
                }
            }
            const bool edge = key_hi > warp_pos_lo ||
                              (window > 0 && key_lo <= warp_pos_hi - window);
            const float* sb = sbias[stage];
            const int d0 = pos_first - key_hi;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key_lo + j * 8 + tq * 2 + (e & 1);
                    const int p = row_pos[e >> 1];
                    float v = (s_acc[j][e] * scale + sb[min(max(p - key - d0, 0), 2 * BN - 1)]) * LOG2E;
                    if (edge) {
                        if (key > p || (window > 0 && key <= p - window && key >= keep_first)) v = -INFINITY;
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
            for (int j = 0; j < BN / 8; ++j) {
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
            for (int kk = 0; kk < BN / 16; ++kk) {
                unsigned pa[4];
                pa[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
                pa[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
                pa[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
                pa[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    unsigned b[4];
                    const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int dim = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + key * ROW_BYTES + dim * 2);
                    mma_bf16(o[2 * dp], pa, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
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
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = warp * 16 + g + 8 * r;
        if (i >= nrows) continue;
        const float inv = 1.0f / l_run[r];
        bf16* op = out + ((size_t)(tok0 + i) * num_heads + h) * HD + tq * 2;
        const float* gp = gate ? gate + (size_t)(tok0 + i) * gate_stride + (size_t)h * HD + tq * 2 : nullptr;
#pragma unroll
        for (int t = 0; t < NT_O; ++t) {
            float a = o[t][2 * r] * inv, b = o[t][2 * r + 1] * inv;
            if (gp) {
                const float2 gv = *reinterpret_cast<const float2*>(gp + t * 8);
                a *= 1.0f / (1.0f + __expf(-gv.x));
                b *= 1.0f / (1.0f + __expf(-gv.y));
            }
            *reinterpret_cast<__nv_bfloat162*>(op + t * 8) = __floats2bfloat162_rn(a, b);
        }
    }
}

// Single-token rows.  A block takes one row and one kv head: the group's query heads are the rows
// of the MMA, and the block's four warps take the tiles of 32 keys in turn (tile i of the walk
// goes to warp i mod 4), each through a two-stage cp.async ring of its own; at the end the warps'
// partial results meet in shared memory, are added in warp order and gated.  The walk and the
// mask are those of the prompt kernel; the bias comes straight from the table.  With few rows the
// walk is cut into `gridDim.z` equal runs, a block each (the count depends on the step's shape
// alone): a block then leaves its unnormalised sums with their maximum and weight in a scratch,
// and attn_bias_decode_merge_kernel adds the runs in order, normalises and gates.
constexpr int DT = 32;
constexpr int DWARPS = 4;

template <int HD>
__global__ void __launch_bounds__(DWARPS * 32)
attn_bias_decode_kernel(const bf16* __restrict__ q, const int* __restrict__ rows,
                        const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                        const int* __restrict__ block_table, int bt_stride,
                        const bf16* __restrict__ pages, int num_pages, int page_size, int num_heads,
                        int num_kv_heads, int window, int keep_first, float scale,
                        const float* __restrict__ dist_bias, int n_dist, const float* gate,
                        int gate_stride, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* __restrict__ status) {
    constexpr int ROW_BYTES = HD * 2 + 16;
    constexpr int CHUNKS = HD / 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    constexpr int WARP_SMEM = 2 * 2 * DT * ROW_BYTES;
    const int nsplit = gridDim.z, split = blockIdx.z;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float sm_m[DWARPS][16], sm_l[DWARPS][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int t = rows[blockIdx.x], kvh = blockIdx.y;
    const int group = num_heads / num_kv_heads;
    const int pos = positions[t], ctx = pos + 1;
    const int* table = block_table + (size_t)req_of_tok[t] * bt_stride;
    const size_t kv_stride = (size_t)num_kv_heads * page_size * HD;
    const int lo = window > 0 ? max(0, ctx - window) : 0;
    const int tile_lo = lo / DT, tile_hi = (ctx + DT - 1) / DT;
    const int n_pre = min(tile_lo, (keep_first + DT - 1) / DT);
    const int n_all = n_pre + (tile_hi - tile_lo);
    const int per_split = (n_all + nsplit - 1) / nsplit;
    const int w_lo = split * per_split, n_walk = min(n_all, w_lo + per_split);   // this block's run of the walk
    auto tile_of = [&](int i) { return i < n_pre ? i : tile_lo + (i - n_pre); };
    unsigned char* mine = smem + (size_t)warp * WARP_SMEM;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    auto issue = [&](int tile, int stage) {
        unsigned char* kdst = mine + (size_t)stage * 2 * DT * ROW_BYTES;
        unsigned char* vdst = kdst + DT * ROW_BYTES;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int key0 = tile * DT + r * 16;
            int pg = -1;
            if (key0 < ctx && (key0 + 16 > lo || key0 < keep_first)) {
                pg = table[key0 / page_size];
                if (pg < 0 || pg >= num_pages) {
                    if (lane == 0) atomicCAS(status, 0, 1);
                    pg = -1;
                }
            }
            const bool valid = pg >= 0;
            const bf16* ksrc = pages;
            if (valid)
                ksrc = pages + (((size_t)pg * 2 * num_kv_heads + kvh) * page_size + key0 % page_size) * HD;
            const bf16* vsrc = valid ? ksrc + kv_stride : pages;
            for (int c = lane; c < 16 * CHUNKS; c += 32) {
                const int off = (r * 16 + c / CHUNKS) * ROW_BYTES + (c % CHUNKS) * 16;
                cp_async16(kdst + off, ksrc + (valid ? c * 8 : 0), valid);
                cp_async16(vdst + off, vsrc + (valid ? c * 8 : 0), valid);
            }
        }
    };

    if (w_lo + warp < n_walk) {
        unsigned qa[KSTEPS][4];
        const bf16* qbase = q + ((size_t)t * num_heads + (size_t)kvh * group) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int k0 = ks * 16 + tq * 2;
            qa[ks][0] = g < group ? *reinterpret_cast<const unsigned*>(qbase + (size_t)g * HD + k0) : 0u;
            qa[ks][1] = g + 8 < group ? *reinterpret_cast<const unsigned*>(qbase + (size_t)(g + 8) * HD + k0) : 0u;
            qa[ks][2] = g < group ? *reinterpret_cast<const unsigned*>(qbase + (size_t)g * HD + k0 + 8) : 0u;
            qa[ks][3] = g + 8 < group ? *reinterpret_cast<const unsigned*>(qbase + (size_t)(g + 8) * HD + k0 + 8) : 0u;
        }
        const float* bias_r[2] = {dist_bias + (size_t)(kvh * group + min(g, group - 1)) * n_dist,
                                  dist_bias + (size_t)(kvh * group + min(g + 8, group - 1)) * n_dist};
        issue(tile_of(w_lo + warp), 0);
        cp_async_commit();
        int turn = 0;
        for (int wi = w_lo + warp; wi < n_walk; wi += DWARPS, ++turn) {
            const int tile = tile_of(wi);
            const int stage = turn & 1;
            if (wi + DWARPS < n_walk) issue(tile_of(wi + DWARPS), stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
            __syncwarp();
            const unsigned char* ks = mine + (size_t)stage * 2 * DT * ROW_BYTES;
            const unsigned char* vs = ks + DT * ROW_BYTES;
            float s_acc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    unsigned b[4];
                    const int key = jp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + key * ROW_BYTES + dim * 2);
                    mma_bf16(s_acc[2 * jp], qa[kk], b[0], b[1]);
                    mma_bf16(s_acc[2 * jp + 1], qa[kk], b[2], b[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = tile * DT + j * 8 + tq * 2 + (e & 1);
                    float v = -INFINITY;
                    if (key < ctx && (key >= lo || key < keep_first))
                        v = (s_acc[j][e] * scale + __ldg(bias_r[e >> 1] + min(pos - key, n_dist - 1))) * LOG2E;
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
                m_use[r] = m_new == -INFINITY ? 0.0f : m_new;
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(s_acc[j][e] - m_use[e >> 1]);
                    s_acc[j][e] = p;
                    sum[e >> 1] += p;
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + sum[r];
#pragma unroll
            for (int i = 0; i < NT_O; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                unsigned pa[4];
                pa[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
                pa[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
                pa[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
                pa[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    unsigned b[4];
                    const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int dim = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + key * ROW_BYTES + dim * 2);
                    mma_bf16(o[2 * dp], pa, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // the warp's partial result takes the place of its tiles: [16 heads][HD] float32
    float* po = reinterpret_cast<float*>(mine);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int i = 0; i < NT_O; ++i)
            *reinterpret_cast<float2*>(po + (g + 8 * r) * HD + i * 8 + tq * 2) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
        if (tq == 0) { sm_m[warp][g + 8 * r] = m_run[r]; sm_l[warp][g + 8 * r] = l_run[r]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += DWARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) mm = fmaxf(mm, sm_m[w][r]);
        float total = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) {
            const float wt = sm_m[w][r] == -INFINITY ? 0.0f : exp2f(sm_m[w][r] - mm);
            total += sm_l[w][r] * wt;
            acc += reinterpret_cast<const float*>(smem + (size_t)w * WARP_SMEM)[r * HD + d] * wt;
        }
        const int head = kvh * group + r;
        if (nsplit > 1) {
            const size_t at = ((size_t)blockIdx.x * num_heads + head) * nsplit + split;
            part_o[at * HD + d] = acc;
            if (d == 0) { part_ml[at * 2] = mm; part_ml[at * 2 + 1] = total; }
            continue;
        }
        float y = acc / total;
        if (gate) y *= 1.0f / (1.0f + __expf(-gate[(size_t)t * gate_stride + (size_t)head * HD + d]));
        out[((size_t)t * num_heads + head) * HD + d] = __float2bfloat16_rn(y);
    }
}

// one block per (row, head), a thread per element: the runs' sums in order
__global__ void attn_bias_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ rows, int num_heads, int hd, int nsplit,
                                              const float* gate, int gate_stride, bf16* __restrict__ out) {
    const int row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    if (d >= hd) return;
    const int t = rows[row];
    const size_t at = ((size_t)row * num_heads + head) * nsplit;
    float mm = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(at + s) * 2]);
    float total = 0.0f, acc = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float m = part_ml[(at + s) * 2];
        const float wt = m == -INFINITY ? 0.0f : exp2f(m - mm);
        total += part_ml[(at + s) * 2 + 1] * wt;
        acc += part_o[(at + s) * hd + d] * wt;
    }
    float y = acc / total;
    if (gate) y *= 1.0f / (1.0f + __expf(-gate[(size_t)t * gate_stride + (size_t)head * hd + d]));
    out[((size_t)t * num_heads + head) * hd + d] = __float2bfloat16_rn(y);
}

template <int HD>
int launch_decode(const bf16* q, const int* rows, int num_rows, const int* positions, const int* req_of_tok,
                  const int* block_table, int bt_stride, const bf16* pages, int num_pages, int page_size,
                  int num_heads, int num_kv_heads, int window, int keep_first, float scale,
                  const float* dist_bias, int n_dist, const float* gate, int gate_stride, bf16* out,
                  int nsplit, float* part_o, float* part_ml, int* status, cudaStream_t s) {
    constexpr int SMEM = DWARPS * 2 * 2 * DT * (HD * 2 + 16);
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_bias_decode_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return ti_fail("attn_bias_decode: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_rows, num_kv_heads, nsplit);
    attn_bias_decode_kernel<HD><<<grid, DWARPS * 32, SMEM, s>>>(
        q, rows, positions, req_of_tok, block_table, bt_stride, pages, num_pages, page_size, num_heads,
        num_kv_heads, window, keep_first, scale, dist_bias, n_dist, gate, gate_stride, out, part_o, part_ml,
        status);
    if (int rc = ti_check_launch("attn_bias_decode")) return rc;
    if (nsplit > 1) {
        attn_bias_decode_merge_kernel<<<dim3(num_rows, num_heads), HD, 0, s>>>(
            part_o, part_ml, rows, num_heads, HD, nsplit, gate, gate_stride, out);
        return ti_check_launch("attn_bias_decode_merge");
    }
    return 0;
}

template <int HD>
int launch_prefill(const bf16* q, const int* tiles, int num_tiles, const int* positions,
                   const int* block_table, int bt_stride, const bf16* pages, int num_pages,
                   int page_size, int num_heads, int num_kv_heads, int window, int keep_first,
                   float scale, const float* dist_bias, int n_dist, const float* gate, int gate_stride,
                   bf16* out, int* status, cudaStream_t s) {
    constexpr int SMEM = STAGES * 2 * BN * (HD * 2 + 16);
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_bias_prefill_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return ti_fail("attn_bias_prefill: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_heads, num_tiles);
    attn_bias_prefill_kernel<HD><<<grid, WARPS * 32, SMEM, s>>>(
        q, tiles, positions, block_table, bt_stride, pages, num_pages, page_size, num_heads, num_kv_heads,
        window, keep_first, scale, dist_bias, n_dist, gate, gate_stride, out, status);
    return ti_check_launch("attn_bias_prefill");
}

}  // namespace

extern "C" int ti_attn_bias_prefill_tile_rows() { return BM; }

extern "C" int ti_attn_bias_prefill_supported(int dk, int dv, int page_size) {
    return dk == dv && dk >= 16 && dk <= 128 && dk % 16 == 0 && page_size >= 16 && page_size % 16 == 0;
}

// tiles: int32 [num_tiles, 3] = {request row, first flat token, query rows}; rows of a tile are
// consecutive tokens of one request.  dist_bias: float32 [num_heads, n_dist]; gate (may be null):
// float32, row t at gate + t * gate_stride, [num_heads * head_dim].
extern "C" int ti_attn_bias_prefill(const void* q, const int* tiles, int num_tiles, const int* positions,
                                    const int* block_table, int bt_stride, const void* pages,
                                    int num_pages, int page_size, int num_heads, int num_kv_heads,
                                    int head_dim, int window, int keep_first, float scale,
                                    const float* dist_bias, int n_dist, const float* gate,
                                    int gate_stride, void* out, int* status, void* stream) {
    if (num_tiles == 0) return 0;
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attn_bias_prefill: %d heads over %d kv heads", num_heads,
               num_kv_heads);
    TI_REQUIRE(ti_attn_bias_prefill_supported(head_dim, head_dim, page_size),
               "attn_bias_prefill: head_dim %d (multiple of 16 up to 128) or page size %d (multiple of 16) "
               "is not supported", head_dim, page_size);
    TI_REQUIRE(num_tiles <= 65535, "attn_bias_prefill: %d tiles exceed the grid limit", num_tiles);
    TI_REQUIRE(dist_bias != nullptr && n_dist >= 1, "attn_bias_prefill: no bias table");
    TI_REQUIRE(gate == nullptr || (gate_stride % 2 == 0 && ((uintptr_t)gate) % 8 == 0),
               "attn_bias_prefill: gate rows must be 8-byte aligned");
#define CASE(HD)                                                                                     \
    case HD:                                                                                         \
        return launch_prefill<HD>((const bf16*)q, tiles, num_tiles, positions, block_table, bt_stride, \
                                  (const bf16*)pages, num_pages, page_size, num_heads, num_kv_heads, \
                                  window, keep_first, scale, dist_bias, n_dist, gate, gate_stride,    \
                                  (bf16*)out, status, (cudaStream_t)stream)
    switch (head_dim) {
        CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    }
#undef CASE
    return ti_fail("attn_bias_prefill: head_dim %d", head_dim);
}

extern "C" int ti_attn_bias_decode_supported(int dk, int dv, int group, int page_size) {
    return dk == dv && dk >= 16 && dk <= 128 && dk % 16 == 0 && group >= 1 && group <= 16 &&
           page_size >= 16 && page_size % 16 == 0;
}

// rows: int32 [num_rows], the flat tokens to compute (each its request's only token of the step).
// nsplit > 1: part_o float32 [num_rows, heads, nsplit, head_dim], part_ml float32 [num_rows, heads, nsplit, 2].
extern "C" int ti_attn_bias_decode(const void* q, const int* rows, int num_rows, const int* positions,
                                   const int* req_of_tok, const int* block_table, int bt_stride,
                                   const void* pages, int num_pages, int page_size, int num_heads,
                                   int num_kv_heads, int head_dim, int window, int keep_first, float scale,
                                   const float* dist_bias, int n_dist, const float* gate, int gate_stride,
                                   void* out, int nsplit, float* part_o, float* part_ml, int* status,
                                   void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || (part_o != nullptr && part_ml != nullptr)),
               "attn_bias_decode: %d runs of keys need a scratch (at most 64)", nsplit);
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attn_bias_decode: %d heads over %d kv heads", num_heads, num_kv_heads);
    TI_REQUIRE(ti_attn_bias_decode_supported(head_dim, head_dim, num_heads / num_kv_heads, page_size),
               "attn_bias_decode: head_dim %d, %d heads per kv head or page size %d is not supported",
               head_dim, num_heads / num_kv_heads, page_size);
    TI_REQUIRE(num_kv_heads <= 65535, "attn_bias_decode: %d kv heads exceed the grid limit", num_kv_heads);
    TI_REQUIRE(dist_bias != nullptr && n_dist >= 1 && rows != nullptr, "attn_bias_decode: no bias table or no rows");
#define CASE(HD)                                                                                      \
    case HD:                                                                                          \
        return launch_decode<HD>((const bf16*)q, rows, num_rows, positions, req_of_tok, block_table,   \
                                 bt_stride, (const bf16*)pages, num_pages, page_size, num_heads,       \
                                 num_kv_heads, window, keep_first, scale, dist_bias, n_dist, gate,     \
                                 gate_stride, (bf16*)out, nsplit, part_o, part_ml, status,             \
                                 (cudaStream_t)stream)
    switch (head_dim) {
        CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    }
#undef CASE
    return ti_fail("attn_bias_decode: head_dim %d", head_dim);
}
