// C++ operator classes with the reference's call shape (constructor, init(), forward()) over the
// operator handles of sdfl.h -- what the reference's nn/GroupNorm, nn/LayerNorm and nn/GEGLU
// classes become when their OpenCL bodies are replaced by libsdfl.so.  Header-only; needs the
// CUDA runtime for the device copies of the weights.
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
// arguments (the reference reads the element count off the cl_mem and is batch-1), and the
// largest tensor forward() will see is stated at construction, because the scratch buffer is
// allocated once in init() and never in forward().
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "sdfl.h"

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
    // max_batch / max_hw / max_dtype: the largest [batch, num_channels, hw] tensor forward() will get.
    GroupNorm(size_t num_groups, size_t num_channels, float eps, std::vector<float> weight,
              std::vector<float> bias, bool fuse_silu = false, int64_t max_batch = 8,
              int64_t max_hw = 512 * 512, int max_dtype = SDFL_F16)
        : num_groups_(num_groups), num_channels_(num_channels), eps_(eps), fuse_silu_(fuse_silu),
          weight_(std::move(weight)), bias_(std::move(bias)), weightSize_(num_channels),
          max_batch_(max_batch), max_hw_(max_hw), max_dtype_(max_dtype) {}
    GroupNorm(const GroupNorm &) = delete;
    GroupNorm &operator=(const GroupNorm &) = delete;
    ~GroupNorm() { sdfl_groupnorm_destroy(op_); }

    void init() {
        if (op_) return;                                                    // GroupNorm.cpp:52-54
        if (weight_.size() != bias_.size())
            throw std::runtime_error("weight.shape[0] != bias.shape[0]");   // GroupNorm.cpp:59-61
        if (weight_.size() != weightSize_)
            throw std::runtime_error("weight.shape[0] != weightSize");      // GroupNorm.cpp:63-65
        bufferWeight_.upload(weight_);
        bufferBias_.upload(bias_);
        const int rc = sdfl_groupnorm_create(&op_, static_cast<int64_t>(num_groups_),
                                             static_cast<int64_t>(num_channels_), eps_,
                                             static_cast<const float *>(bufferWeight_.get()),
                                             static_cast<const float *>(bufferBias_.get()), fuse_silu_ ? 1 : 0,
                                             max_batch_, max_hw_, max_dtype_);
        if (rc == SDFL_ERR_INVALID_VALUE)
            throw std::runtime_error("input_size % weight->num_vals != 0");     // GroupNorm.cpp:83-87
        if (rc != SDFL_OK) throw std::runtime_error(std::string("sdfl_groupnorm_create: ") + sdfl_status_string(rc));
    }

    // input / output: device tensors [batch, num_channels, hw]; output may be input.
    int forward(const void *input, void *output, int64_t batch, int64_t hw, int dtype,
                cudaStream_t stream = nullptr) {
        if (!op_) throw std::runtime_error("GroupNorm::forward before init()");
        return sdfl_groupnorm_op_forward(op_, input, output, batch, hw, dtype, stream);
    }

private:
    size_t num_groups_, num_channels_;
    float eps_;
    bool fuse_silu_;
    std::vector<float> weight_, bias_;
    size_t weightSize_;
    int64_t max_batch_, max_hw_;
    int max_dtype_;
    DeviceBuffer bufferWeight_, bufferBias_;
    sdfl_groupnorm *op_ = nullptr;
};

class LayerNorm {
public:
    LayerNorm(size_t dim, std::vector<float> weight, std::vector<float> bias, float eps = 1e-5f)
        : weightSize_(dim), eps_(eps), weight_(std::move(weight)), bias_(std::move(bias)) {}
    LayerNorm(const LayerNorm &) = delete;
    LayerNorm &operator=(const LayerNorm &) = delete;
    ~LayerNorm() { sdfl_layernorm_destroy(op_); }

    void init() {
        if (op_) return;
        if (weight_.size() != bias_.size()) throw std::runtime_error("weightSize != biasSize");       // LayerNorm.cpp:53-55
        if (weight_.size() != weightSize_) throw std::runtime_error("weightSize != weight->num_vals"); // LayerNorm.cpp:57-59
        bufferWeight_.upload(weight_);
        bufferBias_.upload(bias_);
        const int rc = sdfl_layernorm_create(&op_, static_cast<int64_t>(weightSize_), eps_,
                                             static_cast<const float *>(bufferWeight_.get()),
                                             static_cast<const float *>(bufferBias_.get()));
        if (rc != SDFL_OK) throw std::runtime_error(std::string("sdfl_layernorm_create: ") + sdfl_status_string(rc));
    }

    // input / output: device tensors [rows, dim]; output may be input.
    int forward(const void *input, void *output, int64_t rows, int dtype, cudaStream_t stream = nullptr) {
        if (!op_) throw std::runtime_error("LayerNorm::forward before init()");
        return sdfl_layernorm_op_forward(op_, input, output, rows, dtype, stream);
    }

private:
    size_t weightSize_;
    float eps_;
    std::vector<float> weight_, bias_;
    DeviceBuffer bufferWeight_, bufferBias_;
    sdfl_layernorm *op_ = nullptr;
};

// The gelu_multiply stage of GEGLU::forward (GEGLU.cpp:71-77); the Linear in front of it
// (GEGLU.cpp:32-34) is a dense layer and stays with the caller.
class GEGLU {
public:
    GEGLU(size_t in_features, size_t out_features)
        : weightShape{2 * out_features, in_features}, in_features_(in_features), out_features_(out_features) {}
    GEGLU(const GEGLU &) = delete;
    GEGLU &operator=(const GEGLU &) = delete;
    ~GEGLU() { sdfl_geglu_destroy(op_); }
    void init() {
        if (op_) return;
        const int rc = sdfl_geglu_create(&op_, static_cast<int64_t>(in_features_), static_cast<int64_t>(out_features_));
        if (rc != SDFL_OK) throw std::runtime_error(std::string("sdfl_geglu_create: ") + sdfl_status_string(rc));
    }
    // projected: device [rows, 2 * out_features]; output: device [rows, out_features]
    int forward(const void *projected, void *output, int64_t rows, int dtype, cudaStream_t stream = nullptr) {
        if (!op_) init();
        return sdfl_geglu_op_forward(op_, projected, output, rows, dtype, stream);
    }
    std::vector<size_t> weightShape;                                     // GEGLU.cpp:36

private:
    size_t in_features_, out_features_;
    sdfl_geglu *op_ = nullptr;
};

}  // namespace sdfl_ops
