// Exchange layer for several GPUs (one process and one context per GPU): hash-partitioned
// all-to-all of tuples, small agreement vectors, and the OR of replicated bitmaps, over NCCL.
#pragma once
#include "xlb_ops.h"

constexpr uint32_t COMM_WORDS_MAX = 62;  // longest agreement vector per rank

void comm_destroy(xlb_ctx* c);
bool comm_aborted(const xlb_ctx* c);
// Send every row to the rank that owns the value in half `keysel`; returns the rows this rank
// received (grouped by source rank; sorted and unique when `sorted_unique_result`).
// One collective for the counts, one host wait, one grouped send / receive.
Keys comm_repartition(xlb_ctx* c, const Keys& in, int keysel, bool sorted_unique_result, xlb_run_stats& st);
// Every rank contributes k words and learns all of them: all[r * k + i] = word i of rank r.
// One collective and one host wait; sums, maxima and votes are taken on the host.
void comm_allgather_words(xlb_ctx* c, const uint64_t* mine, uint32_t k, uint64_t* all);
uint64_t comm_allreduce_sum(xlb_ctx* c, uint64_t v);
// The rows of every rank, concatenated in rank order (a bag: callers sort when they need order).
Keys comm_allgather_keys(xlb_ctx* c, const Keys& in);
// bitmap <- OR over all ranks of their bitmaps (`words` 32-bit words each, the same on every rank):
// an all-gather and one pass over the gathered copies; no host wait.
void comm_or_bitmaps(xlb_ctx* c, unsigned int* bitmap, uint64_t words);
// the ranks' bitmaps back to back, in rank order (an all-gather; no host wait)
Buf comm_gather_bitmaps(xlb_ctx* c, const unsigned int* bitmap, uint64_t words);
