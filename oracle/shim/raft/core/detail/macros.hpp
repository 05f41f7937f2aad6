// TEST INFRASTRUCTURE ONLY: stands in for RAFT's macro header when the reference's kernel headers
// are compiled on their own (oracle/ref_search_shim.cu). RAFT is not installed here.
#pragma once
#define RAFT_KERNEL static __global__ void
