// Host-side pieces shared by the model drivers (llama_runner.cu, dekipel_runner.cu): staged checkpoint tensors,
// device allocation helpers, and the slot cache -- the per-task, per-layer row buffers every driver appends to and
// its kernels reach through a device table of slot base pointers (the reference's per-task buffer tables,
// src/model/rag_buffer_context.h:141-181).
#pragma once
#include "common.cuh"

#include <map>
#include <string>
#include <vector>

namespace zl {

#define RCHECK(expr)                  \
    do {                              \
        int _rc = (expr);             \
        if (_rc != ZL_OK) return _rc; \
    } while (0)

inline int dmalloc(void** p, size_t bytes) {
    ZL_CHECK_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    return ZL_OK;
}

// a checkpoint tensor staged on the device until the load pipeline consumes it
struct Staged {
    void* ptr = nullptr;
    int rows = 0, cols = 0, elem = 0;
};
using StagedMap = std::map<std::string, Staged>;

inline const Staged* staged_find(const StagedMap& m, const std::string& name) {
    auto it = m.find(name);
    return it == m.end() ? nullptr : &it->second;
}
inline void staged_drop(StagedMap& m, const std::string& name) {
    auto it = m.find(name);
    if (it != m.end()) {
        cudaFree(it->second.ptr);
        m.erase(it);
    }
}
// copy a host tensor to the device and register it under `name` (replacing an earlier one); synchronous
inline int staged_load(StagedMap& m, const char* name, const void* data_host, int rows, int cols, int elem_bytes,
                       cudaStream_t stream) {
    Staged s;
    s.rows = rows;
    s.cols = cols;
    s.elem = elem_bytes;
    const size_t bytes = (size_t)rows * cols * elem_bytes;
    RCHECK(dmalloc(&s.ptr, bytes));
    ZL_CHECK_CUDA(cudaMemcpyAsync(s.ptr, data_host, bytes, cudaMemcpyHostToDevice, stream));
    ZL_CHECK_CUDA(cudaStreamSynchronize(stream));
    staged_drop(m, name);
    m[name] = s;
    return ZL_OK;
}

// frees device temporaries on every exit path of a load helper
struct DevTmp {
    std::vector<void*> ptrs;
    ~DevTmp() {
        for (void* p : ptrs)
            if (p) cudaFree(p);
    }
    int alloc(void** p, size_t bytes) {
        int rc = dmalloc(p, bytes);
        if (rc == ZL_OK) ptrs.push_back(*p);
        return rc;
    }
};

static __global__ void k_slot_table(void** tab, char* base, size_t stride, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) tab[i] = base + (size_t)i * stride;
}

// One row buffer per slot: (slots, rows_per_slot, row_bytes) in one allocation, zero-filled (rows never written must
// be finite: a masked key still meets an exact 0 weight), plus the device table of the slots' base pointers.  A slot
// that is given to a new sequence needs no clearing: a position is written before any token may see it.
struct SlotCache {
    void* buf = nullptr;
    void** addrs = nullptr;   // device (slots)
    size_t slot_bytes = 0;
    int slots = 0;
    int create(int n_slots, size_t bytes_per_slot, cudaStream_t stream) {
        slots = n_slots;
        slot_bytes = bytes_per_slot;
        RCHECK(dmalloc(&buf, slot_bytes * n_slots));
        ZL_CHECK_CUDA(cudaMemsetAsync(buf, 0, slot_bytes * n_slots, stream));
        RCHECK(dmalloc((void**)&addrs, sizeof(void*) * n_slots));
        k_slot_table<<<cdiv(n_slots, 256), 256, 0, stream>>>(addrs, (char*)buf, slot_bytes, n_slots);
        ZL_CHECK_LAUNCH();
        return ZL_OK;
    }
    void destroy() {
        if (buf) cudaFree(buf);
        if (addrs) cudaFree((void*)addrs);
        buf = nullptr;
        addrs = nullptr;
    }
};

}  // namespace zl
