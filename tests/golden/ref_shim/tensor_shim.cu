// The few members of the reference's Tensor (include/firefly/tensor.h) that its kernel launchers
// use, defined over memory that the caller owns, and a C interface over the reference's own
// launchers (include/firefly/kernels.h).  The kernel sources themselves are compiled unchanged
// from the reference's src/kernels/; this file stands in for src/tensor.cc (which needs <print>
// and the reference's allocators) and adds nothing to the arithmetic.
#include <cuda_runtime.h>

#include "firefly/kernels.h"

namespace firefly
{
Tensor::Tensor(std::vector<int64_t>, DType, Device) { throw std::runtime_error("shim: owning tensors are not built"); }
Tensor::~Tensor() {}
Tensor::Tensor(Tensor&& o) noexcept
    : data_ptr_(o.data_ptr_), shape_(std::move(o.shape_)), strides_(std::move(o.strides_)), numel_(o.numel_),
      dtype_(o.dtype_), device_(o.device_), is_view_(o.is_view_) {}
Tensor Tensor::from_external(void* data_ptr, std::vector<int64_t> shape, DType dtype, Device device)
{
    Tensor t;
    t.data_ptr_ = data_ptr;
    t.shape_ = std::move(shape);
    t.strides_.assign(t.shape_.size(), 1);
    int64_t n = 1;
    for (int i = (int)t.shape_.size() - 1; i >= 0; --i) { t.strides_[i] = n; n *= t.shape_[i]; }
    t.numel_ = n;
    t.dtype_ = dtype;
    t.device_ = device;
    t.is_view_ = true;
    return t;
}
}  // namespace firefly

using firefly::DType;
using firefly::Device;
using firefly::Tensor;
namespace fk = firefly::kernels;

static Tensor ext(void* p, std::vector<int64_t> shape, DType dt = DType::F16)
{
    return Tensor::from_external(p, std::move(shape), dt, Device::CUDA);
}

extern "C" {

int ref_rms_norm(void* x, void* w, void* out, int rows, int width, double eps)
{
    Tensor tx = ext(x, {rows, width}), tw = ext(w, {width}), to = ext(out, {rows, width});
    fk::rms_norm(tx, tw, to, eps);
    return (int)cudaDeviceSynchronize();
}

int ref_rope(void* q, void* k, int batch, int seq_len, int nq, int nkv, int head_dim, float theta, const int* context_lens)
{
    Tensor tq = ext(q, {batch, seq_len, nq, head_dim}), tk = ext(k, {batch, seq_len, nkv, head_dim});
    fk::apply_rope(tq, tk, head_dim, seq_len, theta, context_lens);
    return (int)cudaDeviceSynchronize();
}

int ref_swiglu(void* gate, void* up, void* out, int rows, int width)
{
    Tensor tg = ext(gate, {rows, width}), tu = ext(up, {rows, width}), to = ext(out, {rows, width});
    fk::swiglu(tg, tu, to);
    return (int)cudaDeviceSynchronize();
}

int ref_add_inplace(void* x, void* y, int rows, int width)
{
    Tensor tx = ext(x, {rows, width}), ty = ext(y, {rows, width});
    fk::add_inplace(tx, ty);
    return (int)cudaDeviceSynchronize();
}

int ref_embedding(void* ids, void* table, void* out, int batch, int seq_len, int vocab, int width)
{
    Tensor ti = ext(ids, {batch, seq_len}, DType::I32), tt = ext(table, {vocab, width}),
           to = ext(out, {batch, seq_len, width});
    fk::embedding_lookup(ti, tt, to);
    return (int)cudaDeviceSynchronize();
}

int ref_argmax(void* logits, void* out, int rows, int vocab)
{
    Tensor tl = ext(logits, {rows, vocab}), to = ext(out, {rows}, DType::I32);
    fk::argmax(tl, to);
    return (int)cudaDeviceSynchronize();
}

// The decode branch only (a block table is given): one query token per sequence over the paged
// cache [blocks, 16, nkv, head_dim].
int ref_paged_attention(void* q, void* k_cache, void* v_cache, void* out, void* block_table, int batch, int nq, int nkv,
                        int head_dim, int num_blocks, int max_blocks, const int* context_lens)
{
    if (block_table == nullptr) return -1;
    Tensor tq = ext(q, {batch, 1, nq, head_dim}), tk = ext(k_cache, {num_blocks, 16, nkv, head_dim}),
           tv = ext(v_cache, {num_blocks, 16, nkv, head_dim}), to = ext(out, {batch, 1, nq * head_dim});
    fk::attention(tq, tk, tv, to, block_table, nkv, 1, max_blocks, context_lens);
    return (int)cudaDeviceSynchronize();
}
}
