// Library identity entry points.
#include "common.cuh"

extern "C" int katz_abi_version(void) { return KATZ_ABI_VERSION; }
extern "C" const char* katz_build_arch(void) { return "sm_100a"; }
