#include "umma_launch.h"
namespace fpb {
int launch_umma_bwd(const UmmaBwdArgs&, cudaStream_t, int*) { return FPB_UMMA_NOT_APPLICABLE; }
}
