// Single translation unit of libfastroute_sm100.so.  The parts share one device status
// block, so they are compiled together instead of being device-linked.
#include "fr_route.cu"
#include "fr_route_coop.cu"
#include "fr_gemm.cu"
#include "fr_gemm_tokenn.cu"
#include "fr_w4a16.cu"
#include "fr_ep.cu"
#include "fr_api.cu"
