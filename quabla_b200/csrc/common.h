// Host-side plumbing shared by the translation units of libqb200: status and
// error reporting, the plan description, and the NCCL entry points, which are
// resolved at run time (the reference loads its vendor libraries the same way,
// crates/quabla-core/Cargo.toml:28-30).
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>
#include <vector>

#include "../../include/qb200.h"

namespace qb {

void set_error(const char* fmt, ...);
qb200_status fail(qb200_status status, const char* fmt, ...);

#define QB_CUDA(call)                                                                              \
    do {                                                                                           \
        cudaError_t qb_err__ = (call);                                                             \
        if (qb_err__ != cudaSuccess)                                                               \
            return ::qb::fail(QB200_CUDA_ERROR, "%s failed: %s (%s:%d)", #call,                    \
                              cudaGetErrorString(qb_err__), __FILE__, __LINE__);                   \
    } while (0)

#define QB_TRY(call)                                  \
    do {                                              \
        qb200_status qb_st__ = (call);                \
        if (qb_st__ != QB200_OK) return qb_st__;      \
    } while (0)

struct NcclApi {
    bool loaded = false;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
// Null when libnccl cannot be loaded; the error message says so.
const NcclApi* nccl_api();

}  // namespace qb

struct qb200_desc {
    struct Param {
        std::string name;
        int layer;
        int kind;
    };
    struct Input {
        std::string name;
        int64_t rows, cols;
        bool retained;
    };
    struct Set {
        int64_t n = 0;
        double weight = 0.0;
        std::vector<std::pair<int, int>> cols;  // (input index, column)
        std::vector<std::vector<double>> dirs;
        std::vector<int> orders;
        std::vector<double> merge_w;  // non-empty: one more stream, the weighted sum of second derivatives
        std::vector<int32_t> code;  // 4 per instruction
        std::vector<double> consts;
        int n_regs = 0;
        int value_reg = -1;
        std::vector<int> grad_regs;
        bool has_program = false;
        int streams() const {
            int s = 1;
            for (int k : orders) s += k;
            return s + (merge_w.empty() ? 0 : 1);
        }
    };
    int dtype = QB200_F32;
    int activation = QB200_ACT_TANH;  // of the hidden layers
    std::vector<int> sizes;
    std::vector<Param> params;
    std::vector<Input> inputs;
    std::vector<Set> sets;
};
