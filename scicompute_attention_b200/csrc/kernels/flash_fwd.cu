// Flash prefill entry point (placeholder body until the tcgen05 kernel lands in this file).
#include "common.cuh"

using namespace sca_b200;

extern "C" long long sca_flash_smem_bytes_for(int head_dim, long long elem_bytes, int block_m, int block_n,
                                              int stages) {
    if (head_dim <= 0 || elem_bytes <= 0 || block_m <= 0 || block_n <= 0 || stages <= 0) return -1;
    const long long q = static_cast<long long>(block_m) * head_dim * elem_bytes;
    const long long kv = static_cast<long long>(block_n) * head_dim * elem_bytes * stages;
    return q + 2 * kv + 1024;
}

extern "C" int sca_launch_flash_fwd(const ScaFlashFwdParams* params, void* stream) {
    (void)stream;
    ClearError();
    if (params == nullptr || params->q == nullptr || params->k == nullptr || params->v == nullptr ||
        params->out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: null tensor pointer");
    }
    return Fail(SCA_NOT_IMPLEMENTED, "flash attention: kernel not built yet");
}
