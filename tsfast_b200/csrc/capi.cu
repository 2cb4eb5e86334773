// Entry points that are not tied to one scan: version and workspace status read-back.
#include "common.cuh"

extern "C" {

int b200_version(void) { return 100; }

int b200_workspace_status(const void* workspace, void* stream) {
    if (!workspace) return B200_ERR_ARG;
    b200::WsHeader h;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, st) != cudaSuccess) return B200_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return B200_ERR_LAUNCH;
    return (int)h.error;
}

}  // extern "C"
