// The reference includes the NVTX v2 header name; CUDA 12.9 ships only NVTX v3.
#include <nvtx3/nvToolsExt.h>
