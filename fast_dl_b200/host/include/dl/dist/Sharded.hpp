// dl::dist -- a tensor cut into row blocks over several GPUs of one box, and the path's ops
// on it.  fast_dl has no multi-GPU code; this sits ABOVE dl::ops and leaves dl::Tensor as it
// is (each shard is an ordinary Tensor whose Device carries its GPU index).
//
// Single process, single host thread: an op walks the shards and enqueues the ordinary
// single-GPU op on each shard's device; launches are asynchronous, so the GPUs work
// concurrently.  Elementwise ops, activations, broadcast against a replicated row vector or
// a row-sharded column vector, row reductions, softmax and layernorm need no communication.
// The two ops that do -- the full sum and reductions along axis 0 -- combine one small
// per-GPU partial each, in shard order, so results do not depend on timing.
// (With one PROCESS per GPU the same exchange is done inside the sum kernel over NVLink:
// fdl_sum_allreduce_f32 in include/fdl_kernels.h.)
#pragma once

#include <cstdint>
#include <vector>

#include <dl/tensor/Tensor.hpp>

namespace dl::dist {

class ShardedTensor {
public:
    ShardedTensor() = default;

    /// Cuts `data` (row-major, `shape`) along the leading dimension into one block per entry
    /// of `devices` (CUDA indices; the first `rows % n` blocks get one extra row) and uploads
    /// each block to its GPU.  A device index may appear more than once.
    static ShardedTensor scatter(const std::vector<float>& data, const Shape& shape,
                                 const std::vector<int>& devices);
    /// The same full tensor on every device (row vectors, gamma, beta).
    static ShardedTensor replicate(const std::vector<float>& data, const Shape& shape,
                                   const std::vector<int>& devices);
    /// Wraps per-device results of an op; `global_shape` is the shape of the whole.
    static ShardedTensor from_shards(std::vector<Tensor> shards, const Shape& global_shape, bool replicated);

    /// All shards concatenated along the leading dimension (a replicated tensor: shard 0).
    std::vector<float> gather() const;
    std::vector<int64_t> gather_int64() const;

    const Shape& shape() const { return shape_; }
    int num_shards() const { return static_cast<int>(shards_.size()); }
    bool replicated() const { return replicated_; }
    const Tensor& shard(int i) const { return shards_[static_cast<std::size_t>(i)]; }
    Tensor& shard(int i) { return shards_[static_cast<std::size_t>(i)]; }
    /// First global row of shard i.
    int64_t row_offset(int i) const { return offsets_[static_cast<std::size_t>(i)]; }

private:
    std::vector<Tensor> shards_;
    std::vector<int64_t> offsets_;
    Shape shape_;
    bool replicated_ = false;
};

// ---- shard-local ops: same names and meaning as dl::ops ----
ShardedTensor add(const ShardedTensor& a, const ShardedTensor& b);
ShardedTensor sub(const ShardedTensor& a, const ShardedTensor& b);
ShardedTensor mul(const ShardedTensor& a, const ShardedTensor& b);
ShardedTensor div(const ShardedTensor& a, const ShardedTensor& b);
ShardedTensor mul_add_relu(const ShardedTensor& a, const ShardedTensor& b, const ShardedTensor& c);
ShardedTensor relu(const ShardedTensor& x);
ShardedTensor gelu(const ShardedTensor& x);
ShardedTensor sigmoid(const ShardedTensor& x);
ShardedTensor tanh(const ShardedTensor& x);
ShardedTensor softmax(const ShardedTensor& x);
ShardedTensor layernorm(const ShardedTensor& x, float eps = 1.0e-5f);
ShardedTensor layernorm(const ShardedTensor& x, const ShardedTensor& gamma, const ShardedTensor& beta,
                        float eps = 1.0e-5f);
/// Reductions along the last axis of a rank-2 tensor: the result stays row-sharded.
ShardedTensor sum_rows(const ShardedTensor& x);
ShardedTensor max_rows(const ShardedTensor& x);
ShardedTensor argmax_rows(const ShardedTensor& x);

// ---- ops with an exchange step ----
/// Sum of all elements: one double per GPU, added on the host in shard order.
double sum(const ShardedTensor& x);
/// Mean over the rows of the whole rank-2 tensor, shape [cols], on the first shard's device.
/// Each GPU reduces its rows with the GLOBAL row count as divisor; the per-GPU vectors are
/// added on that device in shard order.
Tensor mean_rows_of_whole(const ShardedTensor& x);

/// Waits for every device that holds a shard.
void synchronize(const ShardedTensor& x);

}  // namespace dl::dist
