// Exchange layer for several GPUs (one process and one context per GPU): hash-partitioned
// all-to-all of tuples and the all-reduced termination vote, over NCCL.
#pragma once
#include "xlb_ops.h"

void comm_destroy(xlb_ctx* c);
// Send every row to the rank that owns the value in half `keysel`; returns the rows this rank
// received (grouped by source rank; sorted and unique when `sorted_unique_result`).
Keys comm_repartition(xlb_ctx* c, const Keys& in, int keysel, bool sorted_unique_result, xlb_run_stats& st);
uint64_t comm_allreduce_sum(xlb_ctx* c, uint64_t v);
