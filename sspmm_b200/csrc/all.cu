// Single translation unit of libsspmm_b200.so: the kernels share file-scope
// device symbols (status words), which needs one TU without relocatable device code.
#include "sspmm_gather.cu"
#include "sspmm_gather_lsu.cu"
#include "sspmm_simt.cu"
#include "sspmm_block.cu"
#include "sspmm_fused.cu"
#include "sspmm_fused_pair.cu"
#include "svc.cu"
#include "c_api.cu"
#include "cxx_api.cu"
#include "sspmm_noalloc.cu"
#include "smtx_io.cu"
#include "reorder.cu"
