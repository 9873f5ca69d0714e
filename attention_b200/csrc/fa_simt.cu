// FlashAttention forward on the FP32 FMA pipe.
//
// This is the exact-arithmetic kernel: every product and sum is FP32 (TF32 tensor cores cannot
// meet a 1e-4 absolute tolerance), inputs of any supported storage type are widened on load and
// the result is rounded to nearest even on store.  It also serves every case the tensor-core
// kernels do not take: head dimensions other than 64/128, strides a tensor map cannot express.
//
// It restates compute_multihead_attention / compute_attention_block of the reference
// (src/algorithms/flash_attention.cpp:277-450) as intended, i.e. with the running (max, sum)
// merge of OnlineSoftmaxState (src/algorithms/flash_attention.hpp:39-62) applied per query row
// and the output accumulator rescaled, not overwritten, between key blocks.
//
// Tiling: one CTA = 64 query rows of one (batch, head); 256 threads as a 16x16 grid, each thread
// owning a 4x4 block of the 64x64 score tile and 4 rows x (DP/16) columns of the output tile.
// Q and K tiles are held transposed in shared memory so the inner product reads are float4 and
// bank-conflict free.  Key tiles wholly above the causal diagonal are skipped.
#include <cmath>

#include "common.cuh"

namespace ahpc {
namespace {

constexpr int BQ = 64;        // query rows per CTA
constexpr int BK = 64;        // keys per tile
constexpr int LDT = 68;       // padded leading dimension of the transposed tiles (float4-aligned)
constexpr int NTHREADS = 256;

template <int DP>
constexpr size_t smem_bytes() {
    // Qt[DP][LDT] + Kt[DP][LDT] + V[BK][DP] + P[BQ][BK+4]
    return sizeof(float) * (size_t(DP) * LDT * 2 + size_t(BK) * DP + size_t(BQ) * (BK + 4));
}

struct SimtParams {
    const void *q, *k, *v;
    void* out;
    const float* mask;
    float* lse;
    int batch, heads, seq_q, seq_kv, head_dim, kv_group;
    int64_t qs[4], ks[4], vs[4], os[4];
    float scale;
    int causal;
    int causal_offset;       // query row r stands at position r + causal_offset
};

template <typename T, int DP>
__global__ void __launch_bounds__(NTHREADS) fa_fwd_simt_kernel(const SimtParams p) {
    extern __shared__ __align__(16) float smem[];
    float* Qt = smem;                        // [DP][LDT]  Qt[d][row]
    float* Kt = Qt + DP * LDT;               // [DP][LDT]  Kt[d][key]
    float* Vs = Kt + DP * LDT;               // [BK][DP]
    float* Ps = Vs + BK * DP;                // [BQ][BK+4]
    constexpr int LDP = BK + 4;
    constexpr int OC = DP / 16;              // output columns per thread

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int b = blockIdx.z, h = blockIdx.y;
    const int q0 = blockIdx.x * BQ;
    const int D = p.head_dim;

    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const int h_kv = h / p.kv_group;                       // grouped-query attention: kv_group query heads share a key/value head
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h_kv * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h_kv * p.vs[1];
    T* og = static_cast<T*>(p.out) + b * p.os[0] + h * p.os[1];

    // Q tile, transposed, zero padded.
    for (int idx = tid; idx < BQ * DP; idx += NTHREADS) {
        int r = idx / DP, d = idx % DP;
        float x = 0.f;
        if (q0 + r < p.seq_q && d < D) x = to_f32<T>(qg[(int64_t)(q0 + r) * p.qs[2] + d * p.qs[3]]);
        Qt[d * LDT + r] = x;
    }

    float m_run[4], l_run[4], acc[4][OC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < OC; ++j) acc[i][j] = 0.f;
    }

    int n_tiles = (p.seq_kv + BK - 1) / BK;
    if (p.causal) {
        // keys beyond the last query row of this tile are all masked
        int last_q = min(q0 + BQ, p.seq_q) - 1 + p.causal_offset;
        n_tiles = min(n_tiles, last_q / BK + 1);
    }

    for (int t = 0; t < n_tiles; ++t) {
        const int k0 = t * BK;
        __syncthreads();   // previous tile's P and V reads are done; Qt is visible on the first pass
        for (int idx = tid; idx < BK * DP; idx += NTHREADS) {
            int r = idx / DP, d = idx % DP;
            float kx = 0.f, vx = 0.f;
            if (k0 + r < p.seq_kv && d < D) {
                kx = to_f32<T>(kg[(int64_t)(k0 + r) * p.ks[2] + d * p.ks[3]]);
                vx = to_f32<T>(vg[(int64_t)(k0 + r) * p.vs[2] + d * p.vs[3]]);
            }
            Kt[d * LDT + r] = kx;
            Vs[r * DP + d] = vx;
        }
        __syncthreads();

        // 4x4 block of raw scores
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 4
        for (int d = 0; d < DP; ++d) {
            float4 qv = *reinterpret_cast<const float4*>(&Qt[d * LDT + ty * 4]);
            float4 kv = *reinterpret_cast<const float4*>(&Kt[d * LDT + tx * 4]);
            const float qa[4] = {qv.x, qv.y, qv.z, qv.w};
            const float ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qa[i], ka[j], s[i][j]);
        }

        // scale, mask, running softmax
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qi = q0 + ty * 4 + i;
            float row_max = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kj = k0 + tx * 4 + j;
                bool visible = qi < p.seq_q && kj < p.seq_kv && !(p.causal && qi + p.causal_offset < kj);
                if (visible && p.mask) visible = p.mask[((int64_t)b * p.seq_q + qi) * p.seq_kv + kj] != 0.0f;
                s[i][j] = visible ? s[i][j] * p.scale : -INFINITY;
                row_max = fmaxf(row_max, s[i][j]);
            }
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, off));
            const float m_new = fmaxf(m_run[i], row_max);
            float row_sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float w = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - m_new);
                row_sum += w;
                Ps[(ty * 4 + i) * LDP + tx * 4 + j] = w;
            }
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, off);
            const float alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
            l_run[i] = l_run[i] * alpha + row_sum;
            m_run[i] = m_new;
#pragma unroll
            for (int j = 0; j < OC; ++j) acc[i][j] *= alpha;
        }
        __syncthreads();

        // acc += P V
#pragma unroll 4
        for (int c = 0; c < BK; ++c) {
            float pv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty * 4 + i) * LDP + c];
#pragma unroll
            for (int j = 0; j < OC; ++j) {
                const float vx = Vs[c * DP + tx + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(pv[i], vx, acc[i][j]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = q0 + ty * 4 + i;
        if (qi >= p.seq_q) continue;
        const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;   // no visible key: zeros
#pragma unroll
        for (int j = 0; j < OC; ++j) {
            const int d = tx + 16 * j;
            if (d < D) og[(int64_t)qi * p.os[2] + d * p.os[3]] = from_f32<T>(acc[i][j] * inv);
        }
        if (p.lse && tx == 0)
            p.lse[((int64_t)b * p.heads + h) * p.seq_q + qi] = l_run[i] > 0.f ? m_run[i] + logf(l_run[i]) : -INFINITY;
    }
}

template <typename T, int DP>
ahpc_status launch_one(const SimtParams& p, cudaStream_t stream) {
    constexpr size_t smem = smem_bytes<DP>();
    static_assert(smem <= 227 * 1024, "tile does not fit in shared memory");
    AHPC_CUDA_OK(cudaFuncSetAttribute(fa_fwd_simt_kernel<T, DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((p.seq_q + BQ - 1) / BQ, p.heads, p.batch);
    fa_fwd_simt_kernel<T, DP><<<grid, NTHREADS, smem, stream>>>(p);
    AHPC_CUDA_OK(cudaGetLastError());
    return AHPC_SUCCESS;
}

template <typename T>
ahpc_status launch_for_dim(const SimtParams& p, cudaStream_t stream) {
    const int D = p.head_dim;
    if (D <= 16) return launch_one<T, 16>(p, stream);
    if (D <= 32) return launch_one<T, 32>(p, stream);
    if (D <= 64) return launch_one<T, 64>(p, stream);
    if (D <= 128) return launch_one<T, 128>(p, stream);
    return launch_one<T, 256>(p, stream);
}

}  // namespace

ahpc_status launch_fa_simt(const FaLaunch& a) {
    if (a.head_dim > 256) return fail(AHPC_UNSUPPORTED_OPERATION, "head_dim %d exceeds 256", a.head_dim);
    if (a.heads > 65535 || a.batch > 65535)
        return fail(AHPC_UNSUPPORTED_OPERATION, "batch (%d) and heads (%d) must not exceed 65535", a.batch, a.heads);
    SimtParams p;
    p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out; p.mask = a.mask; p.lse = a.lse;
    p.batch = a.batch; p.heads = a.heads; p.seq_q = a.seq_q; p.seq_kv = a.seq_kv; p.head_dim = a.head_dim;
    p.kv_group = a.heads / a.kv_heads;
    for (int i = 0; i < 4; ++i) { p.qs[i] = a.qs[i]; p.ks[i] = a.ks[i]; p.vs[i] = a.vs[i]; p.os[i] = a.os[i]; }
    p.scale = a.scale; p.causal = a.causal; p.causal_offset = a.causal_offset;
    switch (a.dtype) {
        case AHPC_F32: return launch_for_dim<float>(p, a.stream);
        case AHPC_F16: return launch_for_dim<__half>(p, a.stream);
        case AHPC_BF16: return launch_for_dim<__nv_bfloat16>(p, a.stream);
    }
    return fail(AHPC_INVALID_PARAMETERS, "unknown dtype %d", a.dtype);
}

}  // namespace ahpc
