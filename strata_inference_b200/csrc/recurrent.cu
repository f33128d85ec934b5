// Mixers that carry a matrix per head from token to token instead of keys and values:
// the gated delta rule (with its short convolutions) and the matrix memory with
// exponential gates.  State, decays, gates, unit norms and the recurrences are 32-bit.
//
// Both recurrences work column by column of the head's matrix S[kd, vd]: column j only
// ever meets v[j], so (head, column) pairs are independent and a launch has
// sequences x heads x columns of parallel work; the tokens of a sequence go one after
// the other.  A column is held in the registers of L neighbouring lanes (32 rows each).
//
//   delta:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//            as one pass:  u = beta (v_j - g <S_j, k>),  o_j = g <S_j, q> + u <k, q>,
//            S_j <- g S_j + u k
//   memory:  m' = max(f + m, i);  a = e^(f + m - m'),  b = e^(i - m');
//            S_j <- a S_j + b v_j k,  o_j = a <S_j, q> + b v_j <k, q>
//            with one more column whose v is 1: it holds n, and its output is <n, q>.
//
// State of a slot: [heads][columns][kd] floats (a column's rows together), then for the
// memory [heads] running maxima.  The delta rule's convolution history lies behind its
// matrices: [taps - 1][channels] floats, oldest first.
//
// Plain counterparts: tests/plain_karupel.py short_conv(), delta_mixer(), mlstm_mixer().
#include "common.cuh"

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) {
    return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}

// ---------------------------------------------------------------------------
// Delta rule, step 1: per row, the short causal convolutions of q | k | v with silu, then
// unit q (times kd^-1/2) and unit k per head, beta and the decay per head.
// ---------------------------------------------------------------------------
struct DeltaPrepareArgs {
    const void* proj;        // [rows, stride]: q (G kd) | k (G kd) | v (H vd) | gate (H vd) | b (H) | a (H)
    const float* conv_w;     // [channels, taps], channels = 2 G kd + H vd, last tap the row's own
    const float* a_log;      // [H]
    const float* dt_bias;    // [H]
    float* state;            // [slots, state_stride]; the history starts at hist_offset
    float* qn;               // [rows, G kd]
    float* kn;               // [rows, G kd]
    float* vc;               // [rows, H vd]
    float* beta;             // [rows, H]
    float* decay;            // [rows, H]
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_row0;
    long long stride, state_stride, hist_offset;
    int H, G, kd, vd, taps;
};

template <typename T>
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepareArgs p) {
    extern __shared__ float conv[];            // [channels] the row's convolved, activated values
    pdl_trigger();
    const int r = blockIdx.x;
    const int nqk = p.G * p.kd, channels = 2 * nqk + p.H * p.vd;
    const int pos = p.row_pos[r];
    const int b = p.row_seq[r];
    const int slot = p.seq_slot[b];
    const int start = p.seq_start[b], row0 = p.seq_row0[b];
    const float* hist = slot >= 0 ? p.state + (size_t)slot * p.state_stride + p.hist_offset : nullptr;
    pdl_wait();
    const T* proj = (const T*)p.proj;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < p.taps; ++j) {
            const int at = pos - (p.taps - 1) + j;      // position of the tap's input
            float x = 0.f;
            if (at >= start) x = to_f32(proj[(size_t)(row0 + at - start) * p.stride + c]);
            else if (hist) x = hist[(size_t)(at - start + p.taps - 1) * channels + c];
            acc += p.conv_w[(size_t)c * p.taps + j] * x;
        }
        conv[c] = silu_f(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int u = warp; u < 2 * p.G; u += warps) {          // q heads, then k heads
        const float* x = conv + (size_t)u * p.kd;
        float ss = 0.f;
        for (int d = lane; d < p.kd; d += 32) ss += x[d] * x[d];
        float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
        if (u < p.G) inv *= 1.0f / sqrtf((float)p.kd);
        float* dst = (u < p.G ? p.qn : p.kn) + (size_t)r * nqk + (size_t)(u % p.G) * p.kd;
        for (int d = lane; d < p.kd; d += 32) dst[d] = x[d] * inv;
    }
    for (int c = threadIdx.x; c < p.H * p.vd; c += blockDim.x)
        p.vc[(size_t)r * p.H * p.vd + c] = conv[2 * nqk + c];
    for (int h = threadIdx.x; h < p.H; h += blockDim.x) {
        const size_t at = (size_t)r * p.stride + channels + (size_t)p.H * p.vd;
        p.beta[(size_t)r * p.H + h] = sigmoid_f(to_f32(proj[at + h]));
        const float dt = softplus_f(to_f32(proj[at + p.H + h]) + p.dt_bias[h]);
        p.decay[(size_t)r * p.H + h] = expf(-expf(p.a_log[h]) * dt);
    }
}

// The history after the step: the last taps - 1 inputs of each sequence.  One thread per
// (sequence, channel) walks the cells oldest first; a cell that keeps an older input takes
// it from a later cell of the same history, which has not been rewritten yet.
template <typename T>
__global__ void conv_history_kernel(const T* __restrict__ proj, long long stride, float* state,
                                    long long state_stride, long long hist_offset,
                                    const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                    const int* __restrict__ seq_end, const int* __restrict__ seq_row0,
                                    int channels, int taps) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int n = seq_end[b] - seq_start[b], row0 = seq_row0[b];
    float* hist = state + (size_t)slot * state_stride + hist_offset;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x)
        for (int i = 0; i < taps - 1; ++i) {
            const int back = taps - 1 - i;              // the input `back` positions before the end
            hist[(size_t)i * channels + c] =
                back <= n ? to_f32(proj[(size_t)(row0 + n - back) * stride + c])
                          : hist[(size_t)(i + n) * channels + c];
        }
}

// ---------------------------------------------------------------------------
// The recurrences.
// ---------------------------------------------------------------------------
enum { SCAN_DELTA = 0, SCAN_MEMORY = 1 };

struct ScanArgs {
    const void* q;           // row r, key head g at q + r * q_stride + g * kd
    const void* k;
    const void* v;           // row r, head h at v + r * v_stride + h * vd
    const float* decay;      // delta: [rows, H]
    const float* beta;       // delta: [rows, H]
    const void* gate_i;      // memory: row r, head h at gate_i + r * gate_stride + h (before bias and cap)
    const void* gate_f;
    const float* bias_i;     // [H]
    const float* bias_f;     // [H]
    float* state;            // [slots, state_stride]
    float* out;              // [rows, H * cols]; cols = vd (delta) or vd + 1 (memory: <n, q> last)
    float* m_out;            // memory: [rows, H] the running maximum after the row
    const int* seq_slot;
    const int* seq_start;
    const int* seq_end;
    const int* seq_row0;
    long long q_stride, k_stride, v_stride, gate_stride, state_stride;
    int H, G, kd, vd;
    float q_scale, cap;
};

constexpr int kPerLane = 32;     // rows of a column that one lane holds

template <typename T> __device__ __forceinline__ void load_slice(const T* src, int d0, int kd,
                                                                  float scale, float (&dst)[kPerLane]) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) dst[i] = d0 + i < kd ? to_f32(src[d0 + i]) * scale : 0.f;
}

template <int L> __device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// blockDim.x threads = blockDim.x / L columns; grid (column tiles, heads, sequences).
template <int MODE, typename TQ, typename TG, int L>
__global__ void __launch_bounds__(64) recurrent_scan_kernel(ScanArgs p) {
    pdl_trigger();
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) / L;
    const int d0 = (threadIdx.x % L) * kPerLane;
    const int h = blockIdx.y, b = blockIdx.z;
    const int cols = MODE == SCAN_MEMORY ? p.vd + 1 : p.vd;
    const bool live = col < cols;          // (idle lanes still take part in the shuffles)
    const int g = h / (p.H / p.G);
    const int slot = p.seq_slot[b];
    const int row0 = p.seq_row0[b], n = p.seq_end[b] - p.seq_start[b];
    float S[kPerLane];
    float* mine = slot >= 0 && live
        ? p.state + (size_t)slot * p.state_stride + ((size_t)h * cols + col) * p.kd : nullptr;
    float* m_cell = MODE == SCAN_MEMORY && slot >= 0
        ? p.state + (size_t)slot * p.state_stride + (size_t)p.H * cols * p.kd + h : nullptr;
    pdl_wait();
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) S[i] = mine && d0 + i < p.kd ? mine[d0 + i] : 0.f;
    float m = m_cell ? *m_cell : 0.f;
    const TQ* qp = (const TQ*)p.q + (size_t)g * p.kd;
    const TQ* kp = (const TQ*)p.k + (size_t)g * p.kd;
    const TQ* vp = (const TQ*)p.v + (size_t)h * p.vd;
    float kk[kPerLane], qq[kPerLane];
    for (int t = 0; t < n; ++t) {
        const size_t r = (size_t)(row0 + t);
        load_slice(kp + r * p.k_stride, d0, p.kd, 1.0f, kk);
        load_slice(qp + r * p.q_stride, d0, p.kd, p.q_scale, qq);
        float vj = 0.f;
        if (live) vj = (MODE == SCAN_MEMORY && col == p.vd) ? 1.0f : to_f32(vp[r * p.v_stride + col]);
        float sk = 0.f, sq = 0.f, kq = 0.f;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            sk += S[i] * kk[i];
            sq += S[i] * qq[i];
            kq += kk[i] * qq[i];
        }
        sq = lanes_sum<L>(sq);
        kq = lanes_sum<L>(kq);
        float keep, take;       // S <- keep S + take k
        if (MODE == SCAN_DELTA) {
            sk = lanes_sum<L>(sk);
            keep = p.decay[r * p.H + h];
            take = p.beta[r * p.H + h] * (vj - keep * sk);
        } else {
            const TG* gi = (const TG*)p.gate_i;
            const TG* gf = (const TG*)p.gate_f;
            const float ig = p.cap * tanhf((to_f32(gi[r * p.gate_stride + h]) + p.bias_i[h]) / p.cap);
            const float fz = p.cap * tanhf((to_f32(gf[r * p.gate_stride + h]) + p.bias_f[h]) / p.cap);
            const float fg = -softplus_f(-fz);             // log sigmoid
            const float m_new = fmaxf(fg + m, ig);
            keep = expf(fg + m - m_new);
            take = expf(ig - m_new) * vj;
            m = m_new;
            if (p.m_out && blockIdx.x == 0 && threadIdx.x == 0) p.m_out[r * p.H + h] = m_new;
        }
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) S[i] = keep * S[i] + take * kk[i];
        if (live && d0 == 0) p.out[(r * p.H + h) * cols + col] = keep * sq + take * kq;
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < kPerLane; ++i)
            if (d0 + i < p.kd) mine[d0 + i] = S[i];
    }
    if (m_cell && blockIdx.x == 0 && threadIdx.x == 0) *m_cell = m;
}

template <int MODE, typename TQ, typename TG>
static int launch_scan(const ScanArgs& p, int n_seqs, cudaStream_t s) {
    const int cols = MODE == SCAN_MEMORY ? p.vd + 1 : p.vd;
    const int L = p.kd <= 32 ? 1 : p.kd <= 64 ? 2 : p.kd <= 128 ? 4 : 8;
    const int threads = 64;
    const dim3 grid((cols * L + threads - 1) / threads, p.H, n_seqs);
#define GO(LL) sib_launch_chained(recurrent_scan_kernel<MODE, TQ, TG, LL>, grid, dim3(threads), 0, s, p)
    if (L == 1) GO(1);
    else if (L == 2) GO(2);
    else if (L == 4) GO(4);
    else GO(8);
#undef GO
    return sib_check_launch("recurrent_scan");
}

static int check_scan(const char* what, int rows, int n_seqs, int H, int G, int kd, int vd) {
    SIB_REQUIRE(rows > 0 && n_seqs > 0 && n_seqs < 65536 && H > 0 && H < 65536 && G > 0 && H % G == 0,
                "%s: rows=%d sequences=%d heads=%d key heads=%d", what, rows, n_seqs, H, G);
    SIB_REQUIRE(kd > 0 && kd <= 8 * kPerLane && vd > 0,
                "%s: key width %d (at most %d) and value width %d", what, kd, 8 * kPerLane, vd);
    return 0;
}

SIB_EXPORT int sib_delta_prepare(
    const void* proj, long long stride, int dtype, const float* conv_w, const float* a_log,
    const float* dt_bias, float* state, long long state_stride, long long hist_offset, float* qn,
    float* kn, float* vc, float* beta, float* decay, const int* row_pos, const int* row_seq,
    const int* seq_slot, const int* seq_start, const int* seq_end, const int* seq_row0, int rows,
    int n_seqs, int H, int G, int kd, int vd, int taps, void* stream) {
    if (rows == 0) return 0;
    if (check_scan("delta_prepare", rows, n_seqs, H, G, kd, vd)) return -1;
    SIB_REQUIRE(taps >= 1 && taps <= 64, "delta_prepare: %d taps", taps);
    const int channels = 2 * G * kd + H * vd;
    const size_t smem = (size_t)channels * sizeof(float);
    SIB_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d channels do not fit shared memory", channels);
    DeltaPrepareArgs p{proj, conv_w, a_log, dt_bias, state, qn, kn, vc, beta, decay, row_pos,
                       row_seq, seq_slot, seq_start, seq_row0, stride, state_stride, hist_offset,
                       H, G, kd, vd, taps};
    cudaStream_t s = (cudaStream_t)stream;
    SIB_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<T>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            SIB_REQUIRE(e == cudaSuccess, "delta_prepare: %s", cudaGetErrorString(e));
        }
        sib_launch_chained(delta_prepare_kernel<T>, dim3(rows), dim3(256), smem, s, p);
    });
    int rc = sib_check_launch("delta_prepare");
    if (rc || taps == 1) return rc;
    const dim3 grid((channels + 255) / 256, n_seqs);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(conv_history_kernel<T>, grid, dim3(256), 0, s,
                                                 (const T*)proj, stride, state, state_stride,
                                                 hist_offset, seq_slot, seq_start, seq_end, seq_row0,
                                                 channels, taps));
    return sib_check_launch("conv_history");
}

SIB_EXPORT int sib_delta_scan(const float* qn, const float* kn, const float* vc, const float* decay,
                              const float* beta, float* state, long long state_stride, float* out,
                              const int* seq_slot, const int* seq_start, const int* seq_end,
                              const int* seq_row0, int rows, int n_seqs, int H, int G, int kd, int vd,
                              void* stream) {
    if (rows == 0) return 0;
    if (check_scan("delta_scan", rows, n_seqs, H, G, kd, vd)) return -1;
    ScanArgs p{qn, kn, vc, decay, beta, nullptr, nullptr, nullptr, nullptr, state, out, nullptr,
               seq_slot, seq_start, seq_end, seq_row0, (long long)G * kd, (long long)G * kd,
               (long long)H * vd, 0, state_stride, H, G, kd, vd, 1.0f, 0.f};
    return launch_scan<SCAN_DELTA, float, float>(p, n_seqs, (cudaStream_t)stream);
}

// q | k | v and the two gates' inputs are columns of one projected row (of `dtype`).
SIB_EXPORT int sib_memory_scan(const void* proj, long long stride, int dtype, long long gate_i_col,
                               long long gate_f_col, const float* bias_i, const float* bias_f,
                               float cap, float* state, long long state_stride, float* out,
                               float* m_out, const int* seq_slot, const int* seq_start,
                               const int* seq_end, const int* seq_row0, int rows, int n_seqs, int H,
                               int kd, int vd, void* stream) {
    if (rows == 0) return 0;
    if (check_scan("memory_scan", rows, n_seqs, H, H, kd, vd)) return -1;
    SIB_REQUIRE(cap > 0.f && bias_i && bias_f, "memory_scan: the gates need a cap and biases");
    const size_t esz = dtype == SIB_F32 ? 4 : 2;
    const char* base = (const char*)proj;
    ScanArgs p{base, base + (size_t)H * kd * esz, base + (size_t)2 * H * kd * esz, nullptr, nullptr,
               base + (size_t)gate_i_col * esz, base + (size_t)gate_f_col * esz, bias_i, bias_f,
               state, out, m_out, seq_slot, seq_start, seq_end, seq_row0, stride, stride, stride,
               stride, state_stride, H, H, kd, vd, 1.0f / sqrtf((float)kd), cap};
    SIB_DISPATCH_DTYPE(dtype, return (launch_scan<SCAN_MEMORY, T, T>(p, n_seqs, (cudaStream_t)stream)));
    return 0;
}

// ---------------------------------------------------------------------------
// After either recurrence: each head's output divided by its root mean square, times a
// weight, times an activated gate.
//   x = o[r, h, :vd]            (memory: divided by max(|o[r, h, vd]|, e^-m[r, h]) + 1e-6)
//   y[r, h, :] = x / sqrt(mean(x^2) + eps) * w[h * w_stride + :] * act(gate[r, h * vd + :])
// act: 0 silu, 1 sigmoid.  One warp per (row, head).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ m, const float* __restrict__ w,
                      int w_stride, const T* __restrict__ gate, long long gate_stride,
                      T* __restrict__ y, int rows, int H, int vd, int cols, float eps, int act) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)rows * H) return;
    const size_t r = unit / H;
    const int h = (int)(unit % H);
    const float* x = o + (size_t)unit * cols;
    float scale = 1.f;
    if (m) scale = 1.0f / (fmaxf(fabsf(x[vd]), expf(-m[unit])) + 1e-6f);
    float ss = 0.f;
    for (int e = lane; e < vd; e += 32) {
        const float v = x[e] * scale;
        ss += v * v;
    }
    const float inv = scale / sqrtf(warp_sum(ss) / (float)vd + eps);
    for (int e = lane; e < vd; e += 32) {
        const float z = to_f32(gate[r * gate_stride + (size_t)h * vd + e]);
        const float a = act == 0 ? silu_f(z) : sigmoid_f(z);
        y[(size_t)unit * vd + e] = from_f32<T>(x[e] * inv * w[(size_t)h * w_stride + e] * a);
    }
}

SIB_EXPORT int sib_head_norm_gate(const float* o, const float* m, const float* w, int w_stride,
                                  const void* gate, long long gate_stride, void* y, int dtype,
                                  int rows, int H, int vd, int cols, float eps, int act,
                                  void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && H > 0 && vd > 0 && cols >= vd && (m == nullptr || cols > vd),
                "head_norm_gate: rows=%d heads=%d width=%d of %d", rows, H, vd, cols);
    const long long blocks = ((long long)rows * H + 3) / 4;
    SIB_REQUIRE(blocks < (1ll << 31), "head_norm_gate: too many rows (%d)", rows);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(head_norm_gate_kernel<T>, dim3((unsigned)blocks),
                                                 dim3(128), 0, (cudaStream_t)stream, o, m, w, w_stride,
                                                 (const T*)gate, gate_stride, (T*)y, rows, H, vd, cols,
                                                 eps, act));
    return sib_check_launch("head_norm_gate");
}
