// placeholder until the tensor-core path lands
#include "context.h"
namespace ormi_b200 {
void gemm_bf16(ormi_b200_ctx*, const GemmArgs&) { throw Error("bf16 tensor-core matmul is not built yet"); }
}
