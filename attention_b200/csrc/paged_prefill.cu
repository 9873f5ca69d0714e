// Prefill over pages: the last n_query[i] tokens of each listed sequence attend to everything the
// pool holds for that sequence (all of it, or - causal - the tokens up to their own position).
//
// The reference reaches this through PagedAttention::forward / forward_batch with more than one
// query token (src/algorithms/paged_attention.cpp:132-174, 496-547, 596-680): it gathers the
// sequence's pages into contiguous buffers and runs the attention loops on them.  Here the
// tensor-core kernel of fa_tc.cu reads the pages where they lie: the TMA producer walks the block
// table, one bulk copy per page of K and one box per page of V.  Pools that kernel cannot take
// (FP32 storage, a page size other than 16, other head sizes, q/out of another type than the pool)
// go through a gather into a staging buffer and the dense kernels.
#include <algorithm>
#include <cmath>
#include <vector>

#include "pool.cuh"

namespace ahpc {
namespace {

struct SeqRun { int seq, first_row, rows, len; };

ahpc_status prefill_by_gather(ahpc_pool* p, const ahpc_prefill_args* a, const std::vector<SeqRun>& runs, int q_heads, float scale,
                              const void* dq, void* dout, int64_t token_stride, int64_t head_stride) {
    // One sequence at a time: K/V out of the pages as [len, kv_heads, D] in the q/out type, then the dense forward.
    const int D = p->cfg.head_dim, kvh = p->cfg.heads;
    const size_t es = dtype_size(a->qo_dtype);
    cudaStream_t st = (cudaStream_t)a->stream;
    for (const SeqRun& r : runs) {
        if (r.rows == 0) continue;
        const size_t kv_bytes = (size_t)r.len * kvh * D * es;
        void *dk = nullptr, *dv = nullptr;
        AHPC_TRY(staging_buffer(p->cfg.device, 9, kv_bytes, &dk));
        AHPC_TRY(staging_buffer(p->cfg.device, 10, kv_bytes, &dv));
        AHPC_TRY(ahpc_pool_gather(p, r.seq, 0, r.len, dk, dv, a->qo_dtype, a->stream));
        FaLaunch l{};
        l.q = static_cast<const char*>(dq) + (size_t)r.first_row * token_stride * es;
        l.out = static_cast<char*>(dout) + (size_t)r.first_row * token_stride * es;
        l.k = dk; l.v = dv; l.mask = nullptr; l.lse = nullptr;
        l.dtype = a->qo_dtype; l.batch = 1; l.heads = q_heads; l.kv_heads = kvh; l.seq_q = r.rows; l.seq_kv = r.len; l.head_dim = D;
        const int64_t qs[4] = {(int64_t)r.rows * q_heads * D, head_stride, token_stride, 1};
        const int64_t ks[4] = {(int64_t)r.len * kvh * D, D, (int64_t)kvh * D, 1};
        for (int i = 0; i < 4; ++i) { l.qs[i] = qs[i]; l.os[i] = qs[i]; l.ks[i] = ks[i]; l.vs[i] = ks[i]; }
        l.scale = scale; l.causal = a->causal != 0; l.causal_offset = r.len - r.rows;
        l.device = p->cfg.device; l.stream = st;
        if (fa_tc_supported(l, nullptr)) AHPC_TRY(launch_fa_tc(l, AHPC_FA_KERNEL_TC_TWO_TILE));
        else AHPC_TRY(launch_fa_simt(l));
        // the staging buffers are reused by the next sequence: same stream, so the order holds
    }
    return AHPC_SUCCESS;
}

}  // namespace
}  // namespace ahpc

using namespace ahpc;

extern "C" ahpc_status ahpc_paged_prefill(const ahpc_prefill_args* a) {
    if (!a || !a->pool) return fail(AHPC_INVALID_INPUT, "ahpc_paged_prefill: NULL argument");
    ahpc_pool* p = a->pool;
    if (a->n_seqs <= 0) return AHPC_SUCCESS;
    if (!a->seqs || !a->n_query) return fail(AHPC_INVALID_INPUT, "ahpc_paged_prefill: seqs and n_query must not be NULL");
    if (!dtype_valid(a->qo_dtype)) return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: unknown dtype %d", a->qo_dtype);
    if (!std::isfinite(a->scale) || a->scale < 0.f) return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: scale must be finite and not negative");
    const int q_heads = a->q_heads > 0 ? a->q_heads : p->cfg.heads;
    if (a->q_heads < 0 || q_heads % p->cfg.heads != 0)
        return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: q_heads (%d) must be a multiple of the pool's heads (%d)", a->q_heads, p->cfg.heads);
    if (a->head_major && a->n_seqs != 1) return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: head_major takes one sequence per call");
    if (a->n_seqs > p->cfg.max_seqs) return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: more sequences (%d) than the pool has slots (%d)", a->n_seqs, p->cfg.max_seqs);

    std::vector<SeqRun> runs((size_t)a->n_seqs);
    long long total_q = 0;
    int max_q = 0;
    bool use_tc = false;
    PagedPrefillLaunch l{};
    const float scale = a->scale != 0.0f ? a->scale : 1.0f / std::sqrt((float)p->cfg.head_dim);
    {
        std::lock_guard<std::mutex> lock(p->mu);
        for (int i = 0; i < a->n_seqs; ++i) {
            const int s = a->seqs[i], n = a->n_query[i];
            if (s < 0 || s >= p->cfg.max_seqs || !p->h_live[s]) return fail(AHPC_INVALID_INPUT, "ahpc_paged_prefill: sequence %d not found", s);
            if (n < 0 || n > p->h_len[s])
                return fail(AHPC_INVALID_PARAMETERS, "ahpc_paged_prefill: %d query tokens for sequence %d, which holds %d", n, s, p->h_len[s]);
            runs[i] = SeqRun{s, (int)total_q, n, p->h_len[s]};
            total_q += n;
            max_q = std::max(max_q, n);
            if (total_q > 2147483647ll) return fail(AHPC_UNSUPPORTED_OPERATION, "ahpc_paged_prefill: more than 2^31-1 query tokens");
        }
    }
    if (total_q == 0) return AHPC_SUCCESS;
    if (!a->q || !a->out) return fail(AHPC_INVALID_INPUT, "ahpc_paged_prefill: q and out must not be NULL");
    ScopedDevice device_guard_(p->cfg.device); AHPC_TRY(device_guard_.status());
    cudaStream_t st = (cudaStream_t)a->stream;

    const size_t qo_bytes = (size_t)total_q * q_heads * p->cfg.head_dim * dtype_size(a->qo_dtype);
    const bool host_q = is_host_pointer(a->q), host_o = is_host_pointer(a->out);
    const void* dq = a->q;
    void* dout = a->out;
    if (host_q) {
        void* s = nullptr;
        AHPC_TRY(staging_buffer(p->cfg.device, 7, qo_bytes, &s));
        AHPC_CUDA_OK(cudaMemcpyAsync(s, a->q, qo_bytes, cudaMemcpyHostToDevice, st));
        dq = s;
    }
    if (host_o) AHPC_TRY(staging_buffer(p->cfg.device, 8, qo_bytes, &dout));

    // [rows, heads, D], or for one sequence [heads, rows, D]
    const int64_t token_stride = a->head_major ? p->cfg.head_dim : (int64_t)q_heads * p->cfg.head_dim;
    const int64_t head_stride = a->head_major ? total_q * p->cfg.head_dim : p->cfg.head_dim;
    l.q = dq; l.out = dout; l.token_stride = token_stride; l.head_stride = head_stride;
    l.dtype = a->qo_dtype == p->cfg.dtype ? a->qo_dtype : -1;
    l.q_heads = q_heads; l.kv_heads = p->cfg.heads; l.head_dim = p->cfg.head_dim; l.page_size = p->cfg.page_size;
    l.total_q = total_q; l.max_q = max_q; l.n_seqs = a->n_seqs;
    l.k_data = p->k_data; l.v_data = p->v_data; l.table = p->table;
    l.page_elems = (long long)p->page_elems; l.num_pages = p->cfg.num_pages; l.max_pages = p->cfg.max_pages_per_seq;
    l.scale = scale; l.causal = a->causal != 0; l.device = p->cfg.device; l.stream = st;
    use_tc = fa_paged_tc_supported(l, nullptr);

    if (use_tc) {
        std::lock_guard<std::mutex> lock(p->mu);
        // {slot, first row, rows, tokens} per listed sequence, into the pool's per-call argument array
        static_assert(sizeof(SeqRun) == sizeof(int4), "SeqRun is read as int4 on the device");
        AHPC_CUDA_OK(cudaMemcpyAsync(p->call_args, runs.data(), runs.size() * sizeof(SeqRun), cudaMemcpyHostToDevice, st));
        l.seqs_dev = reinterpret_cast<const int4*>(p->call_args);
        AHPC_TRY(launch_fa_paged_tc(l));
    } else {
        AHPC_TRY(prefill_by_gather(p, a, runs, q_heads, scale, dq, dout, token_stride, head_stride));
    }
    if (host_o) AHPC_CUDA_OK(cudaMemcpyAsync(a->out, dout, qo_bytes, cudaMemcpyDeviceToHost, st));
    if (host_q || host_o) AHPC_CUDA_OK(cudaStreamSynchronize(st));
    return AHPC_SUCCESS;
}
