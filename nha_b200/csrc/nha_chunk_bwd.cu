#include "nha_common.cuh"
extern "C" int64_t nha_chunk_bwd_workspace_bytes(const nha_chunk_desc* d) { return 0; }
extern "C" int nha_chunk_bwd(const nha_chunk_desc* d, void* stream) { return NHA_ERR_UNSUPPORTED; }
