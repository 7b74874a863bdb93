// The general, node-by-node evaluator of a strongly connected component (any arity up to
// XLB_MAX_ARITY): xlb_tree.cu.  xlb_exec.cu hands it the components its packed pipelines refuse.
#pragma once
#include "xlb_common.cuh"

void run_scc_tree(xlb_ctx* c, const xlb_scc& scc, xlb_run_stats& st);
