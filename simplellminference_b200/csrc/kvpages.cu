// csrc/kvpages.cu — sllm_kvpages_*: the exported face of the page bookkeeping (kvpages.cuh). Its own translation unit so that a
// library holding only part of the kernels can carry it.
#include "kvpages.cuh"

using namespace sllm;

extern "C" {

sllm_kvpages* sllm_kvpages_create(int32_t n_pages, int32_t page_len, int32_t max_seqs, int32_t max_pages_per_seq) {
    if (n_pages < 1 || page_len < 1 || max_seqs < 1 || max_pages_per_seq < 1) {
        set_error("kvpages: n_pages=%d page_len=%d max_seqs=%d max_pages_per_seq=%d must all be positive", n_pages, page_len, max_seqs, max_pages_per_seq);
        return nullptr;
    }
    auto* kp = new sllm_kvpages();
    kp->n_pages = n_pages; kp->page_len = page_len; kp->max_seqs = max_seqs; kp->max_pages = max_pages_per_seq;
    kp->free_.resize(n_pages);
    for (int i = 0; i < n_pages; ++i) kp->free_[i] = n_pages - 1 - i;
    kp->table.assign((size_t)max_seqs * max_pages_per_seq, -1);
    kp->held.assign(max_seqs, 0);
    return kp;
}

void sllm_kvpages_destroy(sllm_kvpages* kp) { delete kp; }

int32_t sllm_kvpages_reserve(sllm_kvpages* kp, int32_t seq, int32_t n_positions) {
    SLLM_REQUIRE(kp && seq >= 0 && seq < kp->max_seqs && n_positions >= 0, SLLM_EINVAL, "kvpages_reserve: bad argument (seq %d, positions %d)", seq, n_positions);
    const int extra = kp->extra_needed(seq, n_positions);
    SLLM_REQUIRE(extra >= 0, SLLM_EINVAL, "kvpages_reserve: %d positions need more than %d pages of %d", n_positions, kp->max_pages, kp->page_len);
    SLLM_REQUIRE(extra <= (int)kp->free_.size(), SLLM_ENOMEM, "out of KV pages: sequence %d needs %d more, %d free", seq, extra, (int)kp->free_.size());
    kp->take(seq, extra);
    return extra;
}

int sllm_kvpages_release(sllm_kvpages* kp, int32_t seq) {
    SLLM_REQUIRE(kp && seq >= 0 && seq < kp->max_seqs, SLLM_EINVAL, "kvpages_release: bad sequence %d", seq);
    kp->release(seq);
    return SLLM_OK;
}

int32_t sllm_kvpages_free_count(const sllm_kvpages* kp) { return kp ? (int32_t)kp->free_.size() : 0; }
int32_t sllm_kvpages_held(const sllm_kvpages* kp, int32_t seq) { return (kp && seq >= 0 && seq < kp->max_seqs) ? kp->held[seq] : 0; }
const int32_t* sllm_kvpages_table(const sllm_kvpages* kp) { return kp ? kp->table.data() : nullptr; }

}  // extern "C"
