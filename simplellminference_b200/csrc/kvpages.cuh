// csrc/kvpages.cuh — host bookkeeping of a paged cache: a stack of free pages and one page list per sequence. Plain host code
// (no device involved), shared by the batched decoder (batch.cu) and the ragged sequence engine (seq_*.cu through the Python face).
#pragma once
#include <algorithm>
#include <vector>

#include "common.cuh"

struct sllm_kvpages {
    int n_pages = 0, page_len = 0, max_seqs = 0, max_pages = 0;
    std::vector<int32_t> free_;    // stack of free page ids; page 0 is handed out first
    std::vector<int32_t> table;    // [max_seqs][max_pages], -1 = none
    std::vector<int32_t> held;     // pages held by each sequence

    int pages_for(int n_positions) const { return (n_positions + page_len - 1) / page_len; }
    // pages a sequence would have to take to cover positions [0, n_positions); < 0: it cannot (beyond max_pages)
    int extra_needed(int seq, int n_positions) const {
        const int need = pages_for(n_positions);
        if (need > max_pages) return -1;
        return std::max(0, need - held[seq]);
    }
    void take(int seq, int extra) {
        for (int i = 0; i < extra; ++i) {
            table[(size_t)seq * max_pages + held[seq]++] = free_.back();
            free_.pop_back();
        }
    }
    void release(int seq) {
        for (int i = held[seq] - 1; i >= 0; --i) {   // so that the pages come back in the order they were handed out
            free_.push_back(table[(size_t)seq * max_pages + i]);
            table[(size_t)seq * max_pages + i] = -1;
        }
        held[seq] = 0;
    }
};

