// Test infrastructure only. Compiles the reference's legacy host-side solver where it lies
// (csrc/kernels/legacy/placement_cpu.cpp, included as a translation unit so that its file-local
// solve_on_host is reachable) and exposes it on host arrays, so that the CPU restatement in
// uep_oracle.cpp can be checked against it without a GPU. REF_LEGACY_CPP is set by the Makefile.
#include REF_LEGACY_CPP

extern "C" void uep_ref_legacy_solve_host(const int32_t* expert_loads, int32_t* p2l, int32_t* l2p, int32_t* lcnts,
                                          int num_logical, int num_ranks, int M, int R, int nvl_ranks, int D,
                                          float balance_threshold) {
    ultra_ep::kernels::legacy::solve_on_host(expert_loads, p2l, l2p, lcnts, num_logical, num_ranks, M, R, nvl_ranks, D,
                                             balance_threshold);
}
