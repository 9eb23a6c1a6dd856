// Sharing one GPU's K/V chunk with the process that drives the neighbouring GPU.
//
// The owner exports a CUDA IPC handle of the allocation that holds the tensor;
// the neighbour opens it WITH ITS OWN DEVICE CURRENT, which maps the memory into
// that device's address space with peer access (cudaIpcMemLazyEnablePeerAccess),
// so kernels launched there can read it over NVLink.  (Opening the handle under
// the owner's device ordinal maps it into a context the neighbour's kernels do
// not run in: such pointers fault when a kernel on the other device touches them.)
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstring>

#include "mat_common.cuh"

using namespace mat;

extern "C" {

int mat_ipc_export(const void *dev_ptr, void *handle_out, int64_t *offset_out) {
    if (!dev_ptr || !handle_out || !offset_out) return fail(MAT_ERR_INVALID, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == MAT_IPC_HANDLE_BYTES, "handle size");
    // the handle names the whole allocation: find its base to report the tensor's offset
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
        return fail(MAT_ERR_CUDA, "cuMemGetAddressRange is not available from this driver");
    CUdeviceptr base = 0;
    size_t size = 0;
    CUresult r = ((PFN_cuMemGetAddressRange_v3020)fn)(&base, &size, (CUdeviceptr)dev_ptr);
    if (r != CUDA_SUCCESS) return fail(MAT_ERR_CUDA, "cuMemGetAddressRange failed with code %d", (int)r);
    cudaIpcMemHandle_t h;
    if ((e = cudaIpcGetMemHandle(&h, (void *)base)) != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
    memcpy(handle_out, &h, sizeof h);
    *offset_out = (int64_t)((CUdeviceptr)dev_ptr - base);
    return MAT_OK;
}

int mat_ipc_open(const void *handle, int device, void **base_out) {
    if (!handle || !base_out) return fail(MAT_ERR_INVALID, "NULL argument");
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "selecting the device");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
    *base_out = p;
    return MAT_OK;
}

int mat_ipc_close(void *base, int device) {
    if (!base) return MAT_OK;
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "selecting the device");
    e = cudaIpcCloseMemHandle(base);
    if (prev != device) cudaSetDevice(prev);
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "cudaIpcCloseMemHandle");
}

}  // extern "C"
