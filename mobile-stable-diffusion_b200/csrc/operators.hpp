// C++ operator classes with the reference's call shape (constructor, init(), forward()) over
// the C ABI of sdfl.h -- what the reference's nn/GroupNorm, nn/LayerNorm and nn/GEGLU classes
// become when their OpenCL bodies are replaced by libsdfl.so.  Header-only; needs the CUDA
// runtime for device memory.
//
// Reference interface (paths inside the reference project, app/src/main/cpp/modules/nn/):
//   GroupNorm.h:15-29   GroupNorm(ctx, queue, num_groups, num_channels, eps, weight_name, bias_name,
//                       kernel); void init(); cl_int forward(in, out, n_wait, wait_list, event)
//   LayerNorm.h:16-28   LayerNorm(ctx, queue, dim, weight_name, bias_name, kernel); same trio
//   GEGLU.h:18-36       GEGLU(ctx, queue, in_features, out_features, ...); same trio
// Kept: argument meaning, init() validating the weights with the reference's messages
// (GroupNorm.cpp:51-66, LayerNorm.cpp:46-64), forward(input, output) with output == input allowed,
// 0 on success, std::runtime_error on contract violations (GroupNorm.cpp:83-93).
// Changed: no OpenCL context / queue / kernel holder (a cudaStream_t per call instead of
// events), weights come as host vectors instead of .npy file names, batch and H*W are
// arguments (the reference reads the element count off the cl_mem and is batch-1).
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/sdfl.h"

namespace sdfl_ops {

inline void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    ~DeviceBuffer() { if (ptr_) cudaFree(ptr_); }
    void reserve(size_t bytes) {
        if (bytes <= bytes_) return;
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
        cuda_check(cudaMalloc(&ptr_, bytes), "cudaMalloc");
        bytes_ = bytes;
    }
    void upload(const std::vector<float> &h) {
        reserve(h.size() * sizeof(float));
        cuda_check(cudaMemcpy(ptr_, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
    }
    void *get() const { return ptr_; }
    size_t bytes() const { return bytes_; }

private:
    void *ptr_ = nullptr;
    size_t bytes_ = 0;
};

class GroupNorm {
public:
    GroupNorm(size_t num_groups, size_t num_channels, float eps, std::vector<float> weight,
              std::vector<float> bias, bool fuse_silu = false)
        : num_groups_(num_groups), num_channels_(num_channels), eps_(eps), fuse_silu_(fuse_silu),
          weight_(std::move(weight)), bias_(std::move(bias)), weightSize_(num_channels) {}

    void init() {
        if (ready_) return;                                              // GroupNorm.cpp:52-54
        if (weight_.size() != bias_.size())
            throw std::runtime_error("weight.shape[0] != bias.shape[0]");   // GroupNorm.cpp:59-61
        if (weight_.size() != weightSize_)
            throw std::runtime_error("weight.shape[0] != weightSize");      // GroupNorm.cpp:63-65
        bufferWeight_.upload(weight_);
        bufferBias_.upload(bias_);
        ready_ = true;
    }

    // input / output: device tensors [batch, num_channels, hw]; output may be input.
    int forward(const void *input, void *output, int64_t batch, int64_t hw, int dtype,
                cudaStream_t stream = nullptr) {
        if (!ready_) throw std::runtime_error("GroupNorm::forward before init()");
        workspace_.reserve(sdfl_groupnorm_workspace_bytes(batch, static_cast<int64_t>(num_channels_), hw,
                                                          static_cast<int64_t>(num_groups_), dtype) + 16);
        const int rc = sdfl_groupnorm_forward(
            input, output, static_cast<const float *>(bufferWeight_.get()),
            static_cast<const float *>(bufferBias_.get()), batch, static_cast<int64_t>(num_channels_), hw,
            static_cast<int64_t>(num_groups_), eps_, fuse_silu_ ? 1 : 0, dtype, workspace_.get(),
            workspace_.bytes(), stream);
        if (rc == SDFL_ERR_INVALID_VALUE)
            throw std::runtime_error("input_size % weight->num_vals != 0");     // GroupNorm.cpp:83-87
        return rc;
    }

private:
    size_t num_groups_, num_channels_;
    float eps_;
    bool fuse_silu_;
    std::vector<float> weight_, bias_;
    size_t weightSize_;
    DeviceBuffer bufferWeight_, bufferBias_, workspace_;
    bool ready_ = false;
};

class LayerNorm {
public:
    LayerNorm(size_t dim, std::vector<float> weight, std::vector<float> bias, float eps = 1e-5f)
        : weightSize_(dim), eps_(eps), weight_(std::move(weight)), bias_(std::move(bias)) {}

    void init() {
        if (ready_) return;
        if (weight_.size() != bias_.size()) throw std::runtime_error("weightSize != biasSize");       // LayerNorm.cpp:53-55
        if (weight_.size() != weightSize_) throw std::runtime_error("weightSize != weight->num_vals"); // LayerNorm.cpp:57-59
        bufferWeight_.upload(weight_);
        bufferBias_.upload(bias_);
        ready_ = true;
    }

    // input / output: device tensors [rows, dim]; output may be input.
    int forward(const void *input, void *output, int64_t rows, int dtype, cudaStream_t stream = nullptr) {
        if (!ready_) throw std::runtime_error("LayerNorm::forward before init()");
        return sdfl_layernorm_forward(input, output, static_cast<const float *>(bufferWeight_.get()),
                                      static_cast<const float *>(bufferBias_.get()), rows,
                                      static_cast<int64_t>(weightSize_), eps_, dtype, stream);
    }

private:
    size_t weightSize_;
    float eps_;
    std::vector<float> weight_, bias_;
    DeviceBuffer bufferWeight_, bufferBias_;
    bool ready_ = false;
};

// The gelu_multiply stage of GEGLU::forward (GEGLU.cpp:71-77); the Linear in front of it
// (GEGLU.cpp:32-34) is a dense layer and stays with the caller.
class GEGLU {
public:
    GEGLU(size_t in_features, size_t out_features)
        : weightShape{2 * out_features, in_features}, out_features_(out_features) {}
    void init() {}
    // projected: device [rows, 2 * out_features]; output: device [rows, out_features]
    int forward(const void *projected, void *output, int64_t rows, int dtype, cudaStream_t stream = nullptr) {
        return sdfl_gelu_multiply(projected, output, rows, static_cast<int64_t>(out_features_), dtype, stream);
    }
    std::vector<size_t> weightShape;                                     // GEGLU.cpp:36

private:
    size_t out_features_;
};

}  // namespace sdfl_ops
