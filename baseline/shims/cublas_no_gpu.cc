// For building the reference's CPU engine on a machine without a GPU: its tensor-resource constructor creates and
// destroys a cuBLAS handle that the CPU path never uses (core/src/executor.cc:34-40), and without a device the real
// cublasCreate leaves the handle unset, so the following cublasDestroy crashes.  These two definitions take the place
// of the library's when (and only when) the CPU-only baseline binary is linked.
extern "C" int cublasCreate_v2(void** handle) { if (handle) *handle = nullptr; return 0; }
extern "C" int cublasDestroy_v2(void*) { return 0; }
