// PyTorch binding: a c10d process-group backend ("nano") and torch ops over the native
// communicator.
//
// No counterpart in the reference (a C++/C library without framework bindings).  Semantics follow
// c10d's CUDA backends: a collective is enqueued on an internal high-priority communication
// stream after everything already queued on the caller's current stream; the returned Work's
// wait() makes the caller's current stream wait for it (no host blocking); tensors are kept
// alive until the communication stream has passed them (recordStream).
//
// Supported: allreduce (sum / avg / max / min; float32, float16, bfloat16), _reduce_scatter_base,
// _allgather_base, allgather and reduce_scatter with tensor lists (through the base forms),
// broadcast (from the root's slot of an AllGather), barrier.  Everything else raises.
#include "gemm/gemm.h"
#include "nano_nccl/communicator.h"

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>
#include <torch/library.h>

#include <atomic>
#include <map>
#include <mutex>

namespace nano_torch {

using nano_nccl::Bootstrap;
using nano_nccl::Communicator;

// Control plane over a c10d::Store: an all-gather is N set()s and N blocking get()s.
class StoreBootstrap final : public Bootstrap {
public:
    StoreBootstrap(c10::intrusive_ptr<c10d::Store> store, int rank, int size, std::string prefix)
        : store_(std::move(store)), rank_(rank), size_(size), prefix_(std::move(prefix)) {}
    int rank() const override { return rank_; }
    int size() const override { return size_; }
    void all_gather(const void* in, void* out, std::size_t bytes) override {
        const std::uint64_t seq = seq_++;
        const auto key = [&](int r) { return prefix_ + "/" + std::to_string(seq) + "/" + std::to_string(r); };
        const auto* p = static_cast<const std::uint8_t*>(in);
        // an empty value is not storable on every Store implementation: pad with one byte
        std::vector<std::uint8_t> mine(p, p + bytes);
        mine.push_back(0);
        store_->set(key(rank_), mine);
        for (int r = 0; r < size_; ++r) {
            const std::vector<std::uint8_t> got = store_->get(key(r));
            TORCH_CHECK(got.size() == bytes + 1, "nano bootstrap: rank ", r, " contributed ", got.size() - 1,
                        " bytes, expected ", bytes);
            if (bytes != 0) std::memcpy(static_cast<char*>(out) + r * bytes, got.data(), bytes);
        }
    }

private:
    c10::intrusive_ptr<c10d::Store> store_;
    int rank_, size_;
    std::string prefix_;
    std::uint64_t seq_ = 0;
};

nano_nccl::DType to_dtype(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return nano_nccl::DType::Float;
        case at::kHalf: return nano_nccl::DType::Float16;
        case at::kBFloat16: return nano_nccl::DType::BFloat16;
        default: TORCH_CHECK(false, "nano backend supports float32, float16 and bfloat16, got ", t);
    }
}

nano_nccl::RedOp to_redop(const c10d::ReduceOp& op) {
    switch (op.op_) {
        case c10d::ReduceOp::SUM: return nano_nccl::RedOp::Sum;
        case c10d::ReduceOp::AVG: return nano_nccl::RedOp::Avg;
        case c10d::ReduceOp::MAX: return nano_nccl::RedOp::Max;
        case c10d::ReduceOp::MIN: return nano_nccl::RedOp::Min;
        default: TORCH_CHECK(false, "nano backend supports sum, avg, max and min reductions");
    }
}

class WorkNano final : public c10d::Work {
public:
    WorkNano(int rank, c10d::OpType type, int device, std::weak_ptr<Communicator> comm)
        : c10d::Work(rank, type), comm_(std::move(comm)), device_(device) {}
    bool isCompleted() override { return event_.query(); }
    // False once the communicator has latched an asynchronous failure (a device wait that ran out, a proxy error).
    bool isSuccess() const override {
        if (auto c = comm_.lock()) {
            try {
                c->check_async_error();
            } catch (const std::exception&) {
                return false;
            }
        }
        return true;
    }
    // Stream semantics: orders the caller's current stream after the collective and returns at once, so the
    // timeout can never run out on the host; a failure that the communicator has latched by now is thrown.
    bool wait(std::chrono::milliseconds /*timeout*/ = kNoTimeout) override {
        if (auto c = comm_.lock()) c->check_async_error();
        event_.block(c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device_)));
        return true;
    }
    void synchronize() override { wait(); }
    std::vector<at::Tensor> result() override { return outputs_; }
    // Completed at enqueue time while the communication stream is current, so the future carries
    // an event on that stream: callbacks and value() consumers are ordered after the collective.
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
    at::cuda::CUDAEvent event_;
    std::vector<at::Tensor> outputs_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;

private:
    std::weak_ptr<Communicator> comm_;  // weak: a pending Work object must not delay the collective teardown
    int device_;
};

class ProcessGroupNano final : public c10d::Backend {
public:
    ProcessGroupNano(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, int device,
                     const std::string& prefix)
        : c10d::Backend(rank, size), device_(device),
          stream_(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, static_cast<c10::DeviceIndex>(device))) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        nano_nccl::CommunicatorConfig cfg;
        cfg.device = device;
        cfg.relaxed_validation = true;
        comm_ = nano_nccl::create_communicator(std::make_shared<StoreBootstrap>(store, rank, size, prefix), cfg);
    }

    const std::string getBackendName() const override { return "nano"; }
    Communicator& communicator() { return *comm_; }

    // Workspace of the fused GEMM + collective kernels, created on first use and re-created when a larger
    // problem arrives.  Collective: every rank calls the fused ops with the same shapes in the same order.
    nano_nccl::FusedGemmContext& fused(std::size_t rs_bytes, std::size_t ag_bytes) {
        if (fused_ == nullptr || rs_bytes > fused_rs_bytes_ || ag_bytes > fused_ag_bytes_) {
            fused_rs_bytes_ = std::max(fused_rs_bytes_, rs_bytes);
            fused_ag_bytes_ = std::max(fused_ag_bytes_, ag_bytes);
            fused_ = std::make_unique<nano_nccl::FusedGemmContext>(*comm_, std::max<std::size_t>(fused_rs_bytes_, 16),
                                                                  std::max<std::size_t>(fused_ag_bytes_, 16));
        }
        return *fused_;
    }
    int device() const { return device_; }

    c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                             const c10d::AllreduceOptions& opts = c10d::AllreduceOptions()) override {
        TORCH_CHECK(tensors.size() == 1, "nano allreduce takes exactly one tensor");
        at::Tensor& t = tensors[0];
        check_tensor(t);
        return run(c10d::OpType::ALLREDUCE, {t}, [&](cudaStream_t s) {
            nano_nccl::AllReduceArgs a;
            a.send_buffer = t.data_ptr();
            a.recv_buffer = t.data_ptr();  // c10d allreduce is in place
            a.stream = s;
            a.count = static_cast<std::size_t>(t.numel());
            a.dtype = to_dtype(t.scalar_type());
            a.redop = to_redop(opts.reduceOp);
            comm_->all_reduce(a);
        });
    }

    c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                        const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override {
        check_tensor(output);
        check_tensor(input);
        TORCH_CHECK(input.numel() == output.numel() * getSize(), "reduce_scatter: input must hold output.numel() * world_size elements");
        return run(c10d::OpType::_REDUCE_SCATTER_BASE, {output, input}, [&](cudaStream_t s) {
            nano_nccl::ReduceScatterArgs a;
            a.send_buffer = input.data_ptr();
            a.recv_buffer = output.data_ptr();
            a.stream = s;
            a.recv_count = static_cast<std::size_t>(output.numel());
            a.dtype = to_dtype(output.scalar_type());
            a.redop = to_redop(opts.reduceOp);
            comm_->reduce_scatter(a);
        });
    }

    // AllGather moves bits, so any dtype is accepted as long as the per-rank byte count is even.
    c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                   const c10d::AllgatherOptions& = c10d::AllgatherOptions()) override {
        check_tensor(output);
        check_tensor(input);
        TORCH_CHECK(output.numel() == input.numel() * getSize() && output.scalar_type() == input.scalar_type(),
                    "all_gather: output must hold input.numel() * world_size elements of the same dtype");
        const std::size_t bytes = static_cast<std::size_t>(input.numel()) * input.element_size();
        TORCH_CHECK(bytes % 2 == 0, "all_gather: per-rank byte count must be even");
        return run(c10d::OpType::_ALLGATHER_BASE, {output, input}, [&](cudaStream_t s) {
            nano_nccl::AllGatherArgs a;
            a.send_buffer = input.data_ptr();
            a.recv_buffer = output.data_ptr();
            a.stream = s;
            const bool words = bytes % 4 == 0 && reinterpret_cast<std::uintptr_t>(input.data_ptr()) % 4 == 0 &&
                               reinterpret_cast<std::uintptr_t>(output.data_ptr()) % 4 == 0;
            a.send_count = words ? bytes / 4 : bytes / 2;
            a.dtype = words ? nano_nccl::DType::Float : nano_nccl::DType::Float16;
            comm_->all_gather(a);
        });
    }

    c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                             const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override {
        TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1 && static_cast<int>(outputs[0].size()) == getSize(),
                    "nano allgather takes one input and world_size outputs");
        at::Tensor flat = at::empty({getSize() * inputs[0].numel()}, inputs[0].options());
        at::Tensor in = inputs[0].contiguous();
        auto work = _allgather_base(flat, in, opts);
        // copy-out on the communication stream, ordered after the collective
        {
            c10::cuda::CUDAStreamGuard g(stream_);
            for (int r = 0; r < getSize(); ++r) {
                outputs[0][r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(outputs[0][r]), true);
                c10::cuda::CUDACachingAllocator::recordStream(outputs[0][r].storage().data_ptr(), stream_);
            }
            static_cast<WorkNano*>(work.get())->event_.record(stream_);
        }
        return work;
    }

    c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                                  const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override {
        TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1 && static_cast<int>(inputs[0].size()) == getSize(),
                    "nano reduce_scatter takes one output and world_size inputs");
        at::Tensor flat = at::cat(inputs[0]).contiguous().view({-1});
        return _reduce_scatter_base(outputs[0], flat, opts);
    }

    c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                             const c10d::BroadcastOptions& opts = c10d::BroadcastOptions()) override {
        TORCH_CHECK(tensors.size() == 1, "nano broadcast takes exactly one tensor");
        at::Tensor& t = tensors[0];
        TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "nano broadcast needs a contiguous CUDA tensor");
        // Any dtype: gather raw bytes (as 2-byte or 4-byte elements) and keep the root's slot.
        const std::size_t bytes = static_cast<std::size_t>(t.numel()) * t.element_size();
        const std::size_t padded = (bytes + 3) / 4 * 4;
        at::Tensor in = at::zeros({static_cast<long>(padded / 4)}, t.options().dtype(at::kFloat));
        at::Tensor all = at::empty({static_cast<long>(padded / 4) * getSize()}, in.options());
        C10_CUDA_CHECK(cudaMemcpyAsync(in.data_ptr(), t.data_ptr(), bytes, cudaMemcpyDeviceToDevice,
                                       c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device_))));
        auto work = _allgather_base(all, in, c10d::AllgatherOptions());
        {
            c10::cuda::CUDAStreamGuard g(stream_);
            C10_CUDA_CHECK(cudaMemcpyAsync(t.data_ptr(), static_cast<char*>(all.data_ptr()) + opts.rootRank * padded, bytes,
                                           cudaMemcpyDeviceToDevice, stream_.stream()));
            c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream_);
            c10::cuda::CUDACachingAllocator::recordStream(all.storage().data_ptr(), stream_);
            static_cast<WorkNano*>(work.get())->event_.record(stream_);
        }
        return work;
    }

    c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& = c10d::BarrierOptions()) override {
        return run(c10d::OpType::BARRIER, {}, [&](cudaStream_t s) { comm_->barrier(s); });
    }

private:
    void check_tensor(const at::Tensor& t) const {
        TORCH_CHECK(t.is_cuda() && t.get_device() == device_, "nano backend: tensor must live on cuda:", device_);
        TORCH_CHECK(t.is_contiguous(), "nano backend: tensor must be contiguous");
        TORCH_CHECK(t.numel() > 0, "nano backend: tensor must not be empty");
    }

    template <typename F>
    c10::intrusive_ptr<c10d::Work> run(c10d::OpType type, std::vector<at::Tensor> tensors, F&& enqueue) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        auto work = c10::make_intrusive<WorkNano>(getRank(), type, device_, comm_);
        // communication stream waits for the producer of the tensors
        at::cuda::CUDAEvent ready;
        ready.record(c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device_)));
        ready.block(stream_);
        enqueue(stream_.stream());
        for (auto& t : tensors) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream_);
        work->event_.record(stream_);
        work->outputs_ = std::move(tensors);
        {
            c10::cuda::CUDAStreamGuard on_comm(stream_);
            work->future_ = c10::make_intrusive<c10::ivalue::Future>(
                c10::ListType::create(c10::TensorType::get()),
                std::vector<c10::Device>{c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device_))});
            work->future_->markCompleted(c10::IValue(work->outputs_));
        }
        return work;
    }

    int device_;
    c10::cuda::CUDAStream stream_;
    std::shared_ptr<Communicator> comm_;
    std::unique_ptr<nano_nccl::FusedGemmContext> fused_;  // after comm_: destroyed before it
    std::size_t fused_rs_bytes_ = 0, fused_ag_bytes_ = 0;
};

// ---------------------------------------------------------------------------- factory + ops
std::atomic<int> g_group_counter{0};
std::mutex g_registry_mutex;
std::map<std::string, c10::intrusive_ptr<ProcessGroupNano>> g_registry;

c10::intrusive_ptr<c10d::Backend> create_process_group(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                       int device, const std::string& name) {
    const std::string prefix = "nano_pg/" + std::to_string(g_group_counter++);
    auto pg = c10::make_intrusive<ProcessGroupNano>(store, rank, size, device, prefix);
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    g_registry[name] = pg;
    return pg;
}

c10::intrusive_ptr<ProcessGroupNano> lookup(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    auto it = g_registry.find(name);
    TORCH_CHECK(it != g_registry.end(), "nano_nccl: no process group named '", name, "'");
    return it->second;
}

void drop_group(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    g_registry.erase(name);
}

c10d::ReduceOp parse_op(const std::string& op) {
    if (op == "sum") return c10d::ReduceOp::SUM;
    if (op == "avg") return c10d::ReduceOp::AVG;
    if (op == "max") return c10d::ReduceOp::MAX;
    if (op == "min") return c10d::ReduceOp::MIN;
    TORCH_CHECK(false, "nano_nccl: unknown reduction '", op, "'");
}

// Functional ops: results are ordered on the caller's current stream when they return.
at::Tensor op_all_reduce(const at::Tensor& input, const std::string& op, const std::string& group) {
    auto pg = lookup(group);
    at::Tensor out = input.contiguous().clone();
    std::vector<at::Tensor> ts{out};
    c10d::AllreduceOptions o;
    o.reduceOp = parse_op(op);
    pg->allreduce(ts, o)->wait();
    return out;
}

at::Tensor op_reduce_scatter(const at::Tensor& input, const std::string& op, const std::string& group) {
    auto pg = lookup(group);
    at::Tensor in = input.contiguous();
    TORCH_CHECK(in.size(0) % pg->getSize() == 0, "reduce_scatter: dim 0 must be divisible by the world size");
    auto sizes = in.sizes().vec();
    sizes[0] /= pg->getSize();
    at::Tensor out = at::empty(sizes, in.options());
    c10d::ReduceScatterOptions o;
    o.reduceOp = parse_op(op);
    pg->_reduce_scatter_base(out, in, o)->wait();
    return out;
}

at::Tensor op_all_gather(const at::Tensor& input, const std::string& group) {
    auto pg = lookup(group);
    at::Tensor in = input.contiguous();
    auto sizes = in.sizes().vec();
    TORCH_CHECK(!sizes.empty(), "all_gather: input needs at least one dimension");
    sizes[0] *= pg->getSize();
    at::Tensor out = at::empty(sizes, in.options());
    pg->_allgather_base(out, in, c10d::AllgatherOptions())->wait();
    return out;
}

void check_bf16_matrix(const at::Tensor& t, const char* what) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.is_contiguous(), "nano_nccl: ", what,
                " must be a contiguous 2-D bfloat16 CUDA tensor");
}

// out[M, N] = a[M, K] @ b[N, K]^T (+ bias[N]): the tcgen05 kernel on the current stream.
at::Tensor op_gemm(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& bias) {
    check_bf16_matrix(a, "a");
    check_bf16_matrix(b, "b");
    TORCH_CHECK(a.size(1) == b.size(1), "nano_nccl.gemm: inner dimensions differ");
    c10::cuda::CUDAGuard guard(a.device());
    at::Tensor out = at::empty({a.size(0), b.size(0)}, a.options());
    const void* bias_ptr = nullptr;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == b.size(0),
                    "nano_nccl.gemm: bias must be a contiguous bfloat16 vector of N elements");
        bias_ptr = bias->data_ptr();
    }
    nano_nccl::gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_ptr, static_cast<int>(a.size(0)),
                         static_cast<int>(b.size(0)), static_cast<int>(a.size(1)),
                         c10::cuda::getCurrentCUDAStream(a.get_device()).stream(), 0);
    return out;
}

// Row-parallel: a[M, K/R] @ w[N, K/R]^T summed over the group, rows scattered: out[M/R, N].  One fused kernel.
at::Tensor op_gemm_rs(const at::Tensor& a, const at::Tensor& w, const std::string& group) {
    auto pg = lookup(group);
    check_bf16_matrix(a, "a");
    check_bf16_matrix(w, "w");
    TORCH_CHECK(a.size(1) == w.size(1), "nano_nccl.gemm_rs: inner dimensions differ");
    TORCH_CHECK(a.size(0) % pg->getSize() == 0, "nano_nccl.gemm_rs: rows must divide by the group size");
    c10::cuda::CUDAGuard guard(a.device());
    const std::size_t rs_bytes = static_cast<std::size_t>(a.size(0)) * static_cast<std::size_t>(w.size(0)) * 2;
    at::Tensor out = at::empty({a.size(0) / pg->getSize(), w.size(0)}, a.options());
    pg->fused(rs_bytes, 0).gemm_rs(a.data_ptr(), w.data_ptr(), out.data_ptr(), static_cast<int>(a.size(0)),
                                   static_cast<int>(w.size(0)), static_cast<int>(a.size(1)),
                                   c10::cuda::getCurrentCUDAStream(a.get_device()).stream());
    return out;
}

// Column-parallel: AllGather(x_shard[M/R, K]) @ w[N/R, K]^T -> out[M, N/R].  One fused kernel.
at::Tensor op_ag_gemm(const at::Tensor& x_shard, const at::Tensor& w, const std::string& group) {
    auto pg = lookup(group);
    check_bf16_matrix(x_shard, "x_shard");
    check_bf16_matrix(w, "w");
    TORCH_CHECK(x_shard.size(1) == w.size(1), "nano_nccl.ag_gemm: inner dimensions differ");
    c10::cuda::CUDAGuard guard(x_shard.device());
    const long m = x_shard.size(0) * pg->getSize();
    const std::size_t ag_bytes = static_cast<std::size_t>(m) * static_cast<std::size_t>(x_shard.size(1)) * 2;
    at::Tensor out = at::empty({m, w.size(0)}, x_shard.options());
    pg->fused(0, ag_bytes).ag_gemm(x_shard.data_ptr(), w.data_ptr(), out.data_ptr(), static_cast<int>(m),
                                   static_cast<int>(w.size(0)), static_cast<int>(x_shard.size(1)),
                                   c10::cuda::getCurrentCUDAStream(x_shard.get_device()).stream(), 0);
    return out;
}

}  // namespace nano_torch

TORCH_LIBRARY(nano_nccl, m) {
    m.def("all_reduce(Tensor input, str op, str group) -> Tensor");
    m.def("reduce_scatter(Tensor input, str op, str group) -> Tensor");
    m.def("all_gather(Tensor input, str group) -> Tensor");
    m.def("gemm(Tensor a, Tensor b, Tensor? bias=None) -> Tensor");
    m.def("gemm_rs(Tensor a, Tensor w, str group) -> Tensor");
    m.def("ag_gemm(Tensor x_shard, Tensor w, str group) -> Tensor");
}

TORCH_LIBRARY_IMPL(nano_nccl, CUDA, m) {
    m.impl("all_reduce", &nano_torch::op_all_reduce);
    m.impl("reduce_scatter", &nano_torch::op_reduce_scatter);
    m.impl("all_gather", &nano_torch::op_all_gather);
    m.impl("gemm", &nano_torch::op_gemm);
    m.impl("gemm_rs", &nano_torch::op_gemm_rs);
    m.impl("ag_gemm", &nano_torch::op_ag_gemm);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("create_process_group", &nano_torch::create_process_group, py::arg("store"), py::arg("rank"), py::arg("size"),
          py::arg("device"), py::arg("name"),
          "Creates the 'nano' c10d backend over a store; registers it under `name` for torch.ops.nano_nccl.*");
    m.def("drop_group", &nano_torch::drop_group);
}
