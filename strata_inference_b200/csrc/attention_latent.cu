// Attention over ONE shared row per position (a latent that is key and value of every head
// at once) on the tensor cores, bfloat16 storage, 32-bit scores, softmax and sums: the prompt
// and the single-token kernel of the latent attention mixer.
//
// A query head h of row r is a vector q[r, h, :kw]; position j of the row's sequence holds one
// row c_j[:kw] (in the step's packed rows, or in the paged cache with one "kv head").  With
//     s_j = scale <q[r, h], c_j>,   visible j: max(0, p - window + 1) <= j <= p  (window 0: all)
//     out[r, h, :] = (sum_j e^{s_j - M} c_j) / (sum_j e^{s_j - M} + e^{sink_h - M})
// every head reads the same rows, so a block takes a tile of up to 16 (row, head) pairs as the
// M side of mma.sync.m16n8k16 and walks the keys 32 at a time: a key tile is fetched ONCE
// (cp.async, two buffers in turn: the next tile is on its way while one is worked on) and
// serves all heads as the B operand of the scores
// (S = Q C^T, the block's 4 warps split kw and add their parts through shared memory) and,
// transposed by ldmatrix, of the weighted sum (O += P C, the warps split the columns).  A tile
// holds 16 heads of one row, or with fewer than 16 heads the heads of several consecutive
// rows; rows of a tile that belong to different sequences are worked on one sequence after
// the other, the others masked.  With splits > 1 a tile's run of keys is cut and the parts
// (max, sum, accumulator) go to scratch memory in the layout of attention_rows.cu, whose
// combine kernel merges them and adds the sink.
//
// The caller keeps the leading columns of `out` that are values (the latent's rank).
// Plain counterpart: tests/plain_vavupel.py latent_attention().
#include "common.cuh"

int sib_launch_attention_combine_sink_bf16(const float* partial, void* out, int units, int splits,
                                           int head_dim, const float* sink, int n_heads,
                                           cudaStream_t s);

namespace {

struct LatentArgs {
    const __nv_bfloat16* q;        // [rows, n_heads * kw]
    const __nv_bfloat16* k_new;    // [rows, kw] of this step (null: keys come from the cache)
    const __nv_bfloat16* k_pool;   // [pages, 1, page_tokens, kw]
    __nv_bfloat16* out;            // [rows, n_heads * kw]
    float* partial;                // [rows, n_heads, splits, kw + 2] when splits > 1
    const float* sink;             // [n_heads] or null
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_row0;
    const int* page_table;
    int rows, n_heads, kw;
    int rpt;                       // rows of a tile (1 with 16 heads or more)
    int head_chunks;               // tiles a row's heads are cut into
    int max_pages, page_tokens, ring_tokens;
    int window, splits;
    float scale;
};

constexpr int KT = 32;             // keys of a tile
constexpr int NKT = KT / 8;        // the tile's groups of 8 keys (N side of the scores)
constexpr int KKT = KT / 16;       // the tile's groups of 16 keys (K side of the weighted sum)
static_assert(KT == 32, "a lane of a warp looks up one row of the tile");
constexpr int STAGES = 2;          // staged tiles
constexpr int PADW = 8;            // bfloat16 elements between the rows of a staged tile

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0: the chunk is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r0), "=r"(r1) : "r"(s));
}
// (not volatile: it touches registers only, so the compiler may place it among the loads)
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// KSW: 16-column steps of kw that one warp multiplies (kw <= 64 KSW); NT: 8-column tiles of
// the output that one warp sums (kw <= 32 NT).
template <int KSW, int NT>
__global__ void __launch_bounds__(128) latent_attention_kernel(LatentArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kw = p.kw, ldk = kw + PADW;
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [STAGES][KT][ldk]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)STAGES * KT * ldk * sizeof(__nv_bfloat16));  // [4][NKT * 4][32]
    const int n_ksteps = kw / 16, n_ntiles = kw / 8;
    const int chunk = blockIdx.x % p.head_chunks;
    const int r0 = (blockIdx.x / p.head_chunks) * p.rpt;
    const int split = blockIdx.y;
    const int rows_here = min(p.rpt, p.rows - r0);
    const int heads_here = min(16, p.n_heads - chunk * 16);
    // the two rows of the M side that this thread holds in accumulators: i0 and i0 + 8
    const int g4 = lane >> 2, q4 = lane & 3;
    int my_row[2], my_head[2];
    bool my_valid[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int i = g4 + 8 * e;
        int rr, hh;
        if (p.rpt == 1) { rr = 0; hh = i; }
        else { rr = i / p.n_heads; hh = i % p.n_heads; }
        my_valid[e] = rr < rows_here && hh < heads_here;
        my_row[e] = r0 + rr;
        my_head[e] = chunk * 16 + hh;
    }
    pdl_wait();
    // this warp's steps of the queries, as A fragments (steps warp, warp + 4, ...)
    uint32_t qa[KSW][4];
#pragma unroll
    for (int s = 0; s < KSW; ++s) {
        const int ks = warp + 4 * s;
#pragma unroll
        for (int e = 0; e < 4; ++e) qa[s][e] = 0u;
        if (ks < n_ksteps) {
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (my_valid[e]) {
                    const __nv_bfloat16* src = p.q + ((size_t)my_row[e] * p.n_heads + my_head[e]) * kw + ks * 16 + 2 * q4;
                    qa[s][e] = *reinterpret_cast<const uint32_t*>(src);
                    qa[s][e + 2] = *reinterpret_cast<const uint32_t*>(src + 8);
                }
        }
    }
    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[t][e] = 0.f;
    // (scores, maxima and the sink in units of log 2, so that a weight is one 2^x)
    constexpr float LOG2E = 1.4426950408889634f;
    const float scale2 = p.scale * LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // one sequence's rows of the tile after the other
    int done = 0;
    while (done < rows_here) {
        const int b = p.row_seq[r0 + done];
        int cnt = 1;
        while (done + cnt < rows_here && p.row_seq[r0 + done + cnt] == b) ++cnt;
        const int slot = p.seq_slot[b], start = p.seq_start[b], row0 = p.seq_row0[b];
        // (rows of one sequence follow one another in position)
        const int pos_first = p.row_pos[r0 + done], pos_last = p.row_pos[r0 + done + cnt - 1];
        const int lo_all = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
        const int span = pos_last - lo_all + 1;
        int per = (span + p.splits - 1) / p.splits;
        per = (per + KT - 1) / KT * KT;
        const int j0 = lo_all + split * per;
        const int j1 = min(j0 + per, pos_last + 1);
        bool act[2];
        int pos[2], lo[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int rr = my_row[e] - r0;
            act[e] = my_valid[e] && rr >= done && rr < done + cnt;
            pos[e] = act[e] ? p.row_pos[my_row[e]] : -1;
            lo[e] = p.window > 0 ? max(0, pos[e] - p.window + 1) : 0;
        }
        const int n_tiles = j1 > j0 ? (j1 - j0 + KT - 1) / KT : 0;
        const int chunks_per_key = kw / 8;
        // Where a tile's 32 rows lie: lane l of every warp looks up row l, one
        // tile ahead of the fetch that uses it, so that the page table's answer has come by
        // then; the lanes then hand the addresses to whichever lane copies a piece of the row.
        auto key_src = [&](int t) -> const __nv_bfloat16* {
            const int j = j0 + t * KT + (lane % KT);
            if (t >= n_tiles || j >= j1) return nullptr;
            if (p.k_new && j >= start) return p.k_new + (size_t)(row0 + (j - start)) * kw;
            const int cell = p.ring_tokens > 0 ? j % p.ring_tokens : j;
            const int page = p.page_table[(size_t)slot * p.max_pages + cell / p.page_tokens];
            return p.k_pool + ((size_t)page * p.page_tokens + cell % p.page_tokens) * kw;
        };
        const __nv_bfloat16* src_next = key_src(0);
        const int pieces = KT * chunks_per_key;
        const int step_key = 128 / chunks_per_key, step_part = 128 % chunks_per_key;
        auto fetch = [&](int t) {          // (called for t = 0, 1, 2, ... in this order)
            __nv_bfloat16* dst = tiles + (size_t)(t % STAGES) * KT * ldk;
            const __nv_bfloat16* src_mine = src_next;
            src_next = key_src(t + 1);
            int key = tid / chunks_per_key, part = tid % chunks_per_key;
            for (int c0 = 0; c0 < pieces; c0 += 128) {
                const bool inside = c0 + tid < pieces;
                const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(
                    __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(src_mine), inside ? key : 0));
                if (inside)      // (a row beyond the run's end is filled with zeros)
                    cp16(dst + (size_t)key * ldk + part * 8, src ? src + part * 8 : p.q, src != nullptr);
                key += step_key;
                part += step_part;
                if (part >= chunks_per_key) { part -= chunks_per_key; ++key; }
            }
            cp_commit();
        };
        if (n_tiles > 0) fetch(0);
        for (int t = 0; t < n_tiles; ++t) {
            if (t + 1 < n_tiles) { fetch(t + 1); cp_wait<1>(); }
            else { cp_wait<0>(); }
            __syncthreads();
            const __nv_bfloat16* kt = tiles + (size_t)(t % STAGES) * KT * ldk;
            // this warp's part of the scores: 16 units x 16 keys
            float s[NKT][4];
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
            for (int sidx = 0; sidx < KSW; ++sidx) {
                const int ks = warp + 4 * sidx;
                if (ks < n_ksteps) {
#pragma unroll
                    for (int n = 0; n < NKT; ++n) {
                        const __nv_bfloat16* bp = kt + (size_t)(n * 8 + g4) * ldk + ks * 16 + 2 * q4;
                        mma16816(s[n], qa[sidx], *reinterpret_cast<const uint32_t*>(bp),
                                 *reinterpret_cast<const uint32_t*>(bp + 8));
                    }
                }
            }
            // (value-major, so that the lanes of a warp touch neighbouring words)
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[(warp * NKT * 4 + n * 4 + e) * 32 + lane] = s[n][e];
            __syncthreads();
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    s[n][e] = (red[(0 * NKT * 4 + n * 4 + e) * 32 + lane] + red[(1 * NKT * 4 + n * 4 + e) * 32 + lane]) +
                              (red[(2 * NKT * 4 + n * 4 + e) * 32 + lane] + red[(3 * NKT * 4 + n * 4 + e) * 32 + lane]);
            // scale (to powers of two), mask, running maximum (per row of the M side: e = 0 holds
            // s[n][0..1], e = 1 s[n][2..3]).  A tile that every row of the warp sees whole
            // skips the mask (a row that is not stored at all may then hold anything finite).
            const int jt = j0 + t * KT;
            bool plain = jt + KT <= j1;
#pragma unroll
            for (int r = 0; r < 2; ++r)
                plain = plain && (!my_valid[r] || (act[r] && lo[r] <= jt && pos[r] >= jt + KT - 1));
            plain = __all_sync(0xffffffffu, plain);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    bool see = true;
                    if (!plain) {
                        const int j = jt + n * 8 + 2 * q4 + (e & 1);
                        see = act[r] && j >= lo[r] && j <= pos[r] && j < j1;
                    }
                    s[n][e] = see ? s[n][e] * scale2 : -INFINITY;
                    mx[r] = fmaxf(mx[r], s[n][e]);
                }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = m_new == -INFINITY ? 1.f : exp2_fast(m_run[r] - m_new);    // (-inf - finite: 0)
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
            float pr[NKT][4];
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    pr[n][e] = m_run[r] == -INFINITY ? 0.f : exp2_fast(s[n][e] - m_run[r]);
                    l_run[r] += pr[n][e];
                }
            const bool rescale = !__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f);
            uint32_t pa[KKT][4];
#pragma unroll
            for (int kk = 0; kk < KKT; ++kk) {
                pa[kk][0] = pack2(pr[2 * kk][0], pr[2 * kk][1]);
                pa[kk][1] = pack2(pr[2 * kk][2], pr[2 * kk][3]);
                pa[kk][2] = pack2(pr[2 * kk + 1][0], pr[2 * kk + 1][1]);
                pa[kk][3] = pack2(pr[2 * kk + 1][2], pr[2 * kk + 1][3]);
            }
            // the weighted sum of this warp's columns (tiles warp, warp + 4, ... of 8 columns);
            // products that follow one another go to different accumulators
            if (rescale) {
#pragma unroll
                for (int ti = 0; ti < NT; ++ti) {
                    o[ti][0] *= corr[0]; o[ti][1] *= corr[0];
                    o[ti][2] *= corr[1]; o[ti][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < KKT; ++kk) {
#pragma unroll
                for (int ti = 0; ti < NT; ++ti) {
                    const int nt = warp + 4 * ti;
                    if (nt < n_ntiles) {
                        uint32_t b0, b1;
                        ldsm_x2_trans(b0, b1, kt + (size_t)(kk * 16 + (lane & 15)) * ldk + nt * 8);
                        mma16816(o[ti], pa[kk], b0, b1);
                    }
                }
            }
            __syncthreads();       // (the tile's buffer is fetched into again at the start of the tile after the next)
        }
        done += cnt;
    }
    // the sums of a row over the four threads that hold its columns
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (p.splits == 1) {
        float inv[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float scale_o = 1.f, l = l_run[r];
            if (p.sink && my_valid[r]) {
                const float sk = p.sink[my_head[r]] * LOG2E;
                const float top = fmaxf(m_run[r], sk);
                scale_o = m_run[r] == -INFINITY ? 0.f : exp2_fast(m_run[r] - top);
                l = l * scale_o + exp2_fast(sk - top);
            }
            inv[r] = l > 0.f ? scale_o / l : 0.f;
        }
#pragma unroll
        for (int ti = 0; ti < NT; ++ti) {
            const int nt = warp + 4 * ti;
            if (nt >= n_ntiles) continue;
#pragma unroll
            for (int r = 0; r < 2; ++r)
                if (my_valid[r]) {
                    __nv_bfloat16* dst = p.out + ((size_t)my_row[r] * p.n_heads + my_head[r]) * kw + nt * 8 + 2 * q4;
                    *reinterpret_cast<uint32_t*>(dst) = pack2(o[ti][2 * r] * inv[r], o[ti][2 * r + 1] * inv[r]);
                }
        }
    } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (!my_valid[r]) continue;
            float* pp = p.partial + (((size_t)my_row[r] * p.n_heads + my_head[r]) * p.splits + split) * (kw + 2);
            // (the combine kernel takes maxima in natural units)
            if (warp == 0 && q4 == 0) { pp[0] = m_run[r] * (1.0f / LOG2E); pp[1] = l_run[r]; }
#pragma unroll
            for (int ti = 0; ti < NT; ++ti) {
                const int nt = warp + 4 * ti;
                if (nt < n_ntiles)
                    *reinterpret_cast<float2*>(pp + 2 + nt * 8 + 2 * q4) = make_float2(o[ti][2 * r], o[ti][2 * r + 1]);
            }
        }
    }
}

}  // namespace

SIB_EXPORT int sib_attention_latent_supports(int n_heads, int kw) {
    return n_heads > 0 && kw >= 16 && kw % 16 == 0 && kw <= 512;
}

SIB_EXPORT int sib_attention_latent(
    const void* q, const void* k_new, const void* k_pool, const int* page_table, int max_pages,
    int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq, const int* seq_slot,
    const int* seq_start, const int* seq_row0, void* out, float* partial, const float* sink, int rows,
    int n_heads, int kw, float scale, int window, int splits, int rows_per_tile, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && sib_attention_latent_supports(n_heads, kw),
                "attention_latent: rows=%d heads=%d row width=%d (a multiple of 16 up to 512)", rows,
                n_heads, kw);
    SIB_REQUIRE(k_new != nullptr || (k_pool && page_table && page_tokens > 0 && max_pages > 0),
                "attention_latent: no keys given, or an incomplete cache description");
    SIB_REQUIRE(splits >= 1 && splits < 65536 && (splits == 1 || partial != nullptr),
                "attention_latent: splits=%d without scratch memory", splits);
    SIB_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_new % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 &&
                    ((uintptr_t)out % 4) == 0,
                "attention_latent: rows must start on 16-byte boundaries");
    SIB_REQUIRE(window >= 0 && ring_tokens >= 0, "attention_latent: window=%d ring=%d", window, ring_tokens);
    const int rpt = n_heads >= 16 ? 1 : (rows_per_tile < 1 ? 1 : (rows_per_tile * n_heads > 16 ? 16 / n_heads : rows_per_tile));
    const int head_chunks = (n_heads + 15) / 16;
    LatentArgs p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)k_pool,
                 (__nv_bfloat16*)out, partial, sink, row_pos, row_seq, seq_slot, seq_start, seq_row0,
                 page_table, rows, n_heads, kw, rpt, head_chunks, max_pages, page_tokens, ring_tokens,
                 window, splits, scale};
    const long long tiles = (long long)((rows + rpt - 1) / rpt) * head_chunks;
    SIB_REQUIRE(tiles < (1ll << 31), "attention_latent: too many rows (%d)", rows);
    const dim3 grid((unsigned)tiles, (unsigned)splits);
    const size_t smem = (size_t)STAGES * KT * (kw + PADW) * sizeof(__nv_bfloat16) + (size_t)4 * NKT * 4 * 32 * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define GO(KSW, NT)                                                                                \
    do {                                                                                           \
        if (smem > 48 * 1024) {                                                                    \
            cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<KSW, NT>,                 \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            SIB_REQUIRE(e == cudaSuccess, "attention_latent: %s", cudaGetErrorString(e));          \
        }                                                                                          \
        sib_launch_chained(latent_attention_kernel<KSW, NT>, grid, dim3(128), smem, s, p);         \
    } while (0)
    if (kw <= 64) GO(1, 2);
    else if (kw <= 128) GO(2, 4);
    else if (kw <= 256) GO(4, 8);
    else GO(8, 16);
#undef GO
    int rc = sib_check_launch("attention_latent");
    if (rc || splits == 1) return rc;
    return sib_launch_attention_combine_sink_bf16((const float*)partial, out, rows * n_heads, splits, kw,
                                                  sink, n_heads, s);
}
