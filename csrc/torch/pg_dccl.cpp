/**
 * PyTorch process-group backend "dccl": c10d::Backend on top of the library's
 * public API (include/dccl/dccl.hpp).
 *
 * CPU tensors go through the shared-memory host path and complete before the
 * call returns. CUDA tensors are launched on a communication stream owned by
 * the backend: the stream first waits for the caller's current stream, the
 * collective kernel is enqueued, and the returned Work carries an event; wait()
 * makes the caller's current stream wait for that event (the host never
 * blocks), and getFuture() gives DDP the future it needs to overlap bucketed
 * gradient all-reduce with the rest of backward.
 *
 * The rendezvous token of the library travels through the c10d Store, so
 * init_process_group(backend="dccl") needs nothing beyond what torchrun sets.
 */
#include <torch/python.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#define DCCL_WITH_CUDA_RUNTIME 1
#include <dccl/dccl.hpp>

#include <atomic>
#include <cstring>
#include <memory>
#include <mutex>

namespace {

using c10d::Work;

dccl::ncclDataType_t to_dtype(at::ScalarType t) {
    switch (t) {
    case at::kChar: return dccl::ncclInt8;
    case at::kByte: case at::kBool: return dccl::ncclUint8;
    case at::kInt: return dccl::ncclInt32;
    case at::kLong: return dccl::ncclInt64;
    case at::kHalf: return dccl::ncclFloat16;
    case at::kFloat: return dccl::ncclFloat32;
    case at::kDouble: return dccl::ncclFloat64;
    case at::kBFloat16: return dccl::ncclBfloat16;
    case at::kUInt32: return dccl::ncclUint32;
    case at::kUInt64: return dccl::ncclUint64;
    default: TORCH_CHECK(false, "dccl backend: unsupported dtype ", t);
    }
}

dccl::ncclRedOp_t to_op(const c10d::ReduceOp& op) {
    switch (op.op_) {
    case c10d::ReduceOp::SUM: return dccl::ncclSum;
    case c10d::ReduceOp::PRODUCT: return dccl::ncclProd;
    case c10d::ReduceOp::MAX: return dccl::ncclMax;
    case c10d::ReduceOp::MIN: return dccl::ncclMin;
    case c10d::ReduceOp::AVG: return dccl::ncclAvg;
    default: TORCH_CHECK(false, "dccl backend: unsupported reduce operation");
    }
}

void check(dccl::ncclResult_t r, const char* what) {
    TORCH_CHECK(r == dccl::ncclSuccess, "dccl backend: ", what, " failed: ", dccl::dcclGetErrorString(r));
}

class WorkDccl : public Work {
public:
    WorkDccl(c10d::OpType op, std::vector<at::Tensor> outputs, bool cuda, dccl::ncclComm_t comm = nullptr)
        : Work(-1, op), outputs_(std::move(outputs)), cuda_(cuda), comm_(comm) {
        if (cuda_) {
            event_ = std::make_shared<at::cuda::CUDAEvent>(cudaEventDisableTiming);
            std::vector<c10::Device> devs;
            if (!outputs_.empty()) devs.push_back(outputs_[0].device());
            future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devs);
        } else {
            future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
        }
    }
    /** Called right after the kernel was enqueued on `stream` (CUDA) or the host call returned (CPU). */
    void launched(const c10::cuda::CUDAStream* stream) {
        if (cuda_) {
            event_->record(*stream);
            // the future records its own events on the current stream, which must be the communication stream here
            c10::cuda::CUDAStreamGuard g(*stream);
            future_->markCompleted(c10::IValue(outputs_));
        } else {
            future_->markCompleted(c10::IValue(outputs_));
        }
        finish();
    }
    bool isCompleted() override { return !cuda_ || event_->query(); }
    /** What the communicator knows by now: a bounded wait inside a kernel that gave up, or an abort by the watchdog,
     *  shows in its status block (the kernels of later calls may not have run yet; they report through later work). */
    bool isSuccess() const override {
        if (!comm_) return true;
        dccl::ncclResult_t async = dccl::ncclSuccess;
        char msg[160];
        dccl::dcclGetLastError(comm_, &async, msg, sizeof(msg));
        return async == dccl::ncclSuccess;
    }
    bool wait(std::chrono::milliseconds = std::chrono::milliseconds(0)) override {
        synchronize();
        if (comm_) {
            dccl::ncclResult_t async = dccl::ncclSuccess;
            char msg[160] = "";
            dccl::dcclGetLastError(comm_, &async, msg, sizeof(msg));
            TORCH_CHECK(async == dccl::ncclSuccess, "dccl backend: the communicator reported ", dccl::dcclGetErrorString(async), ": ", msg);
        }
        return true;
    }
    void synchronize() override {
        if (cuda_ && !outputs_.empty()) {
            auto cur = c10::cuda::getCurrentCUDAStream(outputs_[0].device().index());
            event_->block(cur);
        }
    }
    std::vector<at::Tensor> result() override { return outputs_; }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

private:
    std::vector<at::Tensor> outputs_;
    bool cuda_;
    dccl::ncclComm_t comm_;
    std::shared_ptr<at::cuda::CUDAEvent> event_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class BackendDccl : public c10d::Backend {
public:
    BackendDccl(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size) : Backend(rank, size) {
        // The store is private to the process group (c10d prefixes it per group and device), so the key only has to
        // tell apart several backends made on the same store: every member counts its own creations there, and all
        // members of a group create the same number. (A counter of the process would run apart between ranks as soon
        // as subgroups with different members exist.)
        const int64_t instance = store->add("dccl_instances/" + std::to_string(rank), 1);
        const std::string key = "dccl_unique_id/" + std::to_string(instance);
        dccl::dcclUniqueId id;
        if (rank == 0) {
            check(dccl::dcclGetUniqueId(&id), "dcclGetUniqueId");
            std::vector<uint8_t> v(sizeof(id));
            memcpy(v.data(), &id, sizeof(id));
            store->set(key, v);
        } else {
            std::vector<uint8_t> v = store->get(key);
            TORCH_CHECK(v.size() == sizeof(id), "dccl backend: bad rendezvous token in the store");
            memcpy(&id, v.data(), sizeof(id));
        }
        check(dccl::dcclCommInitRank(&comm_, size, id, rank), "dcclCommInitRank");
    }
    ~BackendDccl() override { shutdown(); }
    void shutdown() override {
        std::lock_guard<std::mutex> g(mu_);
        if (comm_) {
            try { dccl::ncclCommFinalize(comm_); } catch (...) {}
            comm_ = nullptr;
        }
    }
    void abort() override { if (comm_) dccl::dcclCommAbort(comm_); }
    const std::string getBackendName() const override { return "dccl"; }

    /* ---- collectives ---- */
    c10::intrusive_ptr<Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override {
        at::Tensor& t = one(tensors);
        return run(c10d::OpType::ALLREDUCE, {t}, t, [&](cudaStream_t s) {
            return dccl::ncclAllReduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), to_op(opts.reduceOp), comm_, s);
        });
    }
    c10::intrusive_ptr<Work> allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) override {
        TORCH_CHECK(!tensors.empty(), "dccl backend: empty tensor list");
        for (auto& t : tensors) TORCH_CHECK(t.is_contiguous(), "dccl backend: tensors must be contiguous");
        return run(c10d::OpType::ALLREDUCE_COALESCED, tensors, tensors[0], [&](cudaStream_t s) {
            for (auto& t : tensors) {
                auto r = dccl::ncclAllReduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), to_op(opts.reduceOp), comm_, s);
                if (r != dccl::ncclSuccess) return r;
            }
            return dccl::ncclSuccess;
        });
    }
    c10::intrusive_ptr<Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override {
        at::Tensor& t = one(tensors);
        return run(c10d::OpType::BROADCAST, {t}, t, [&](cudaStream_t s) {
            return dccl::ncclBroadcast(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), (int)opts.rootRank, comm_, s);
        });
    }
    c10::intrusive_ptr<Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override {
        at::Tensor& t = one(tensors);
        return run(c10d::OpType::REDUCE, {t}, t, [&](cudaStream_t s) {
            return dccl::ncclReduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), to_op(opts.reduceOp), (int)opts.rootRank, comm_, s);
        });
    }
    c10::intrusive_ptr<Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions&) override {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "dccl backend: tensors must be contiguous");
        TORCH_CHECK(out.numel() == in.numel() * getSize(), "dccl backend: all_gather output must hold world_size inputs");
        return run(c10d::OpType::_ALLGATHER_BASE, {out}, out, [&](cudaStream_t s) {
            return dccl::ncclAllGather(in.data_ptr(), out.data_ptr(), (size_t)in.numel(), to_dtype(in.scalar_type()), comm_, s);
        }, false, nullptr, {in});
    }
    c10::intrusive_ptr<Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions& opts) override {
        TORCH_CHECK(ins.size() == 1 && outs.size() == 1 && (int)outs[0].size() == getSize(), "dccl backend: all_gather expects one input and world_size outputs");
        at::Tensor in = ins[0].contiguous();
        at::Tensor flat = at::empty({(int64_t)getSize() * in.numel()}, in.options());
        auto w = _allgather_base(flat, in, opts);
        // the copies into the caller's list run on the communication stream too, before the event the caller waits on
        return run(c10d::OpType::ALLGATHER, outs[0], in, [&](cudaStream_t) {
            for (int r = 0; r < getSize(); r++) outs[0][r].copy_(flat.narrow(0, (int64_t)r * in.numel(), in.numel()).view_as(outs[0][r]), true);
            return dccl::ncclSuccess;
        }, /*torch_ops=*/true, w);
    }
    c10::intrusive_ptr<Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions& opts) override {
        TORCH_CHECK(outs.size() == ins.size(), "dccl backend: mismatched lists");
        c10::intrusive_ptr<Work> w;
        for (size_t i = 0; i < ins.size(); i++) w = _allgather_base(outs[i], ins[i], opts);
        return w;
    }
    c10::intrusive_ptr<Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in, const c10d::ReduceScatterOptions& opts) override {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "dccl backend: tensors must be contiguous");
        TORCH_CHECK(in.numel() == out.numel() * getSize(), "dccl backend: reduce_scatter input must hold world_size outputs");
        return run(c10d::OpType::_REDUCE_SCATTER_BASE, {out}, out, [&](cudaStream_t s) {
            return dccl::ncclReduceScatter(in.data_ptr(), out.data_ptr(), (size_t)out.numel(), to_dtype(in.scalar_type()), to_op(opts.reduceOp), comm_, s);
        }, false, nullptr, {in});
    }
    c10::intrusive_ptr<Work> reduce_scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ReduceScatterOptions& opts) override {
        TORCH_CHECK(outs.size() == 1 && ins.size() == 1 && (int)ins[0].size() == getSize(), "dccl backend: reduce_scatter expects one output and world_size inputs");
        std::vector<at::Tensor> flat_parts;
        for (auto& t : ins[0]) flat_parts.push_back(t.reshape({-1}));
        at::Tensor flat = at::cat(flat_parts);
        at::Tensor out = outs[0];
        TORCH_CHECK(out.is_contiguous(), "dccl backend: tensors must be contiguous");
        return _reduce_scatter_base(out, flat, opts);
    }
    c10::intrusive_ptr<Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::ReduceScatterOptions& opts) override {
        TORCH_CHECK(outs.size() == ins.size(), "dccl backend: mismatched lists");
        c10::intrusive_ptr<Work> w;
        for (size_t i = 0; i < ins.size(); i++) w = _reduce_scatter_base(outs[i], ins[i], opts);
        return w;
    }
    c10::intrusive_ptr<Work> send(std::vector<at::Tensor>& tensors, int dst, int) override {
        at::Tensor& t = one(tensors);
        return run(c10d::OpType::SEND, {t}, t, [&](cudaStream_t s) {
            return dccl::ncclSend(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), dst, comm_, s);
        });
    }
    c10::intrusive_ptr<Work> recv(std::vector<at::Tensor>& tensors, int src, int) override {
        at::Tensor& t = one(tensors);
        return run(c10d::OpType::RECV, {t}, t, [&](cudaStream_t s) {
            return dccl::ncclRecv(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), src, comm_, s);
        });
    }
    c10::intrusive_ptr<Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& out_splits, std::vector<int64_t>& in_splits,
                                           const c10d::AllToAllOptions&) override {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "dccl backend: tensors must be contiguous");
        TORCH_CHECK(out.scalar_type() == in.scalar_type(), "dccl backend: all_to_all tensors must have one dtype");
        const int n = getSize();
        // splits count rows of dimension 0; a row is numel / size(0) elements
        const size_t in_row = in.dim() > 0 && in.size(0) > 0 ? (size_t)(in.numel() / in.size(0)) : 1;
        const size_t out_row = out.dim() > 0 && out.size(0) > 0 ? (size_t)(out.numel() / out.size(0)) : 1;
        std::vector<size_t> sc((size_t)n), sd((size_t)n), rc((size_t)n), rd((size_t)n);
        if (in_splits.empty()) {
            TORCH_CHECK(in.numel() % n == 0, "dccl backend: all_to_all input must divide by the world size");
            for (int p = 0; p < n; p++) sc[(size_t)p] = (size_t)in.numel() / (size_t)n;
        } else {
            TORCH_CHECK((int)in_splits.size() == n, "dccl backend: one input split per rank");
            for (int p = 0; p < n; p++) sc[(size_t)p] = (size_t)in_splits[(size_t)p] * in_row;
        }
        if (out_splits.empty()) {
            TORCH_CHECK(out.numel() % n == 0, "dccl backend: all_to_all output must divide by the world size");
            for (int p = 0; p < n; p++) rc[(size_t)p] = (size_t)out.numel() / (size_t)n;
        } else {
            TORCH_CHECK((int)out_splits.size() == n, "dccl backend: one output split per rank");
            for (int p = 0; p < n; p++) rc[(size_t)p] = (size_t)out_splits[(size_t)p] * out_row;
        }
        size_t so = 0, ro = 0;
        for (int p = 0; p < n; p++) { sd[(size_t)p] = so; so += sc[(size_t)p]; rd[(size_t)p] = ro; ro += rc[(size_t)p]; }
        TORCH_CHECK(so <= (size_t)in.numel() && ro <= (size_t)out.numel(), "dccl backend: splits exceed the tensors");
        if (in_splits.empty() && out_splits.empty() && in.numel() == out.numel() && in.numel() % n == 0)
            return run(c10d::OpType::ALLTOALL_BASE, {out}, out, [&](cudaStream_t s) {
                return dccl::dcclAllToAll(in.data_ptr(), out.data_ptr(), (size_t)in.numel() / (size_t)n, to_dtype(in.scalar_type()), comm_, s);
            }, false, nullptr, {in});
        return run(c10d::OpType::ALLTOALL_BASE, {out}, out, [&](cudaStream_t s) {
            return dccl::dcclAllToAllv(in.data_ptr(), sc.data(), sd.data(), out.data_ptr(), rc.data(), rd.data(), to_dtype(in.scalar_type()), comm_, s);
        }, false, nullptr, {in});
    }
    c10::intrusive_ptr<Work> alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllToAllOptions&) override {
        const int n = getSize(), me = getRank();
        TORCH_CHECK((int)outs.size() == n && (int)ins.size() == n, "dccl backend: all_to_all expects world_size tensors on both sides");
        for (int p = 0; p < n; p++) TORCH_CHECK(outs[(size_t)p].is_contiguous() && ins[(size_t)p].is_contiguous(), "dccl backend: tensors must be contiguous");
        return run(c10d::OpType::ALLTOALL, outs, outs[0], [&](cudaStream_t s) {
            dccl::ncclResult_t res = dccl::ncclSuccess;
            dccl::dcclGroupStart();
            for (int k = 1; k < n && res == dccl::ncclSuccess; k++) {
                at::Tensor& t = outs[(size_t)((me - k + n) % n)];
                if (t.numel()) res = dccl::ncclRecv(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), (me - k + n) % n, comm_, s);
            }
            for (int k = 1; k < n && res == dccl::ncclSuccess; k++) {
                at::Tensor& t = ins[(size_t)((me + k) % n)];
                if (t.numel()) res = dccl::ncclSend(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), (me + k) % n, comm_, s);
            }
            dccl::ncclResult_t e = dccl::dcclGroupEnd();
            if (res == dccl::ncclSuccess) res = e;
            if (res == dccl::ncclSuccess) outs[(size_t)me].copy_(ins[(size_t)me], true);
            return res;
        }, /*torch_ops=*/true, nullptr, ins);
    }
    c10::intrusive_ptr<Work> gather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::GatherOptions& opts) override {
        const int n = getSize(), me = getRank(), root = (int)opts.rootRank;
        at::Tensor& in = one(ins);
        if (me == root) TORCH_CHECK(outs.size() == 1 && (int)outs[0].size() == n, "dccl backend: the root of gather needs world_size outputs");
        if (me == root)
            for (auto& t : outs[0]) TORCH_CHECK(t.is_contiguous() && t.numel() == in.numel(), "dccl backend: gather outputs must be contiguous and of the input's size");
        std::vector<at::Tensor> results = me == root ? outs[0] : std::vector<at::Tensor>{};
        return run(c10d::OpType::GATHER, results, in, [&](cudaStream_t s) {
            if (me != root) return dccl::ncclSend(in.data_ptr(), (size_t)in.numel(), to_dtype(in.scalar_type()), root, comm_, s);
            dccl::ncclResult_t res = dccl::ncclSuccess;
            dccl::dcclGroupStart();
            for (int p = 0; p < n && res == dccl::ncclSuccess; p++) {
                if (p == root) continue;
                at::Tensor& t = outs[0][(size_t)p];
                res = dccl::ncclRecv(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), p, comm_, s);
            }
            dccl::ncclResult_t e = dccl::dcclGroupEnd();
            if (res == dccl::ncclSuccess) res = e;
            if (res == dccl::ncclSuccess) outs[0][(size_t)root].copy_(in, true);
            return res;
        }, /*torch_ops=*/true, nullptr, {in});
    }
    c10::intrusive_ptr<Work> scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ScatterOptions& opts) override {
        const int n = getSize(), me = getRank(), root = (int)opts.rootRank;
        at::Tensor& out = one(outs);
        if (me == root) TORCH_CHECK(ins.size() == 1 && (int)ins[0].size() == n, "dccl backend: the root of scatter needs world_size inputs");
        if (me == root)
            for (auto& t : ins[0]) TORCH_CHECK(t.is_contiguous() && t.numel() == out.numel(), "dccl backend: scatter inputs must be contiguous and of the output's size");
        return run(c10d::OpType::SCATTER, {out}, out, [&](cudaStream_t s) {
            if (me != root) return dccl::ncclRecv(out.data_ptr(), (size_t)out.numel(), to_dtype(out.scalar_type()), root, comm_, s);
            dccl::ncclResult_t res = dccl::ncclSuccess;
            dccl::dcclGroupStart();
            for (int p = 0; p < n && res == dccl::ncclSuccess; p++) {
                if (p == root) continue;
                at::Tensor& t = ins[0][(size_t)p];
                res = dccl::ncclSend(t.data_ptr(), (size_t)t.numel(), to_dtype(t.scalar_type()), p, comm_, s);
            }
            dccl::ncclResult_t e = dccl::dcclGroupEnd();
            if (res == dccl::ncclSuccess) res = e;
            if (res == dccl::ncclSuccess) out.copy_(ins[0][(size_t)root], true);
            return res;
        }, /*torch_ops=*/true, nullptr, me == root ? ins[0] : std::vector<at::Tensor>{});
    }
    /* ---- coalescing (torch.distributed.batch_isend_irecv): sends and receives issued between start and end are
     *      recorded and leave as ONE grouped launch, so a ring of isend / irecv cannot deadlock ---- */
    bool supportsCoalescing() const override { return true; }
    void startCoalescing() override {
        std::lock_guard<std::mutex> g(mu_);
        TORCH_CHECK(!coalescing_, "dccl backend: coalescing is already active");
        check(dccl::dcclGroupStart(), "dcclGroupStart");
        coalescing_ = true;
        coalesced_device_ = -1;
    }
    c10::intrusive_ptr<Work> endCoalescing() override {
        std::lock_guard<std::mutex> g(mu_);
        TORCH_CHECK(coalescing_, "dccl backend: endCoalescing without startCoalescing");
        coalescing_ = false;
        const dccl::ncclResult_t r = dccl::dcclGroupEnd();     // device operations launch on the communication stream here
        check(r, "dcclGroupEnd");
        const bool cuda = coalesced_device_ >= 0;
        auto work = c10::make_intrusive<WorkDccl>(c10d::OpType::COALESCED, std::vector<at::Tensor>{}, cuda);
        if (cuda) {
            c10::cuda::CUDAGuard dg((c10::DeviceIndex)coalesced_device_);
            work->launched(&comm_stream((c10::DeviceIndex)coalesced_device_));
        } else work->launched(nullptr);
        return work;
    }
    c10::intrusive_ptr<Work> barrier(const c10d::BarrierOptions&) override {
        // What this rank has queued on the communication stream finishes first; then a host all-reduce of one word,
        // which returns when every rank has arrived: after the barrier every rank's earlier collectives are complete.
        {
            std::lock_guard<std::mutex> g(mu_);
            if (stream_) stream_->synchronize();
        }
        int32_t word = 0;
        check(dccl::ncclAllReduce(&word, &word, 1, dccl::ncclInt32, dccl::ncclSum, comm_, nullptr), "barrier");
        auto w = c10::make_intrusive<WorkDccl>(c10d::OpType::BARRIER, std::vector<at::Tensor>{}, false);
        w->launched(nullptr);
        return w;
    }

    dccl::ncclComm_t comm() const { return comm_; }

    static c10::intrusive_ptr<c10d::Backend> create(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, double /*timeout_s*/) {
        return c10::make_intrusive<BackendDccl>(store, rank, size);
    }

private:
    static at::Tensor& one(std::vector<at::Tensor>& tensors) {
        TORCH_CHECK(tensors.size() == 1, "dccl backend: expected exactly one tensor");
        TORCH_CHECK(tensors[0].is_contiguous(), "dccl backend: tensors must be contiguous");
        return tensors[0];
    }

    c10::cuda::CUDAStream& comm_stream(c10::DeviceIndex dev) {
        if (!stream_ || stream_->device_index() != dev) stream_ = std::make_unique<c10::cuda::CUDAStream>(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, dev));
        return *stream_;
    }

    /** `keep`: inputs that the communication stream reads; like the outputs they must not be handed back to the
     *  allocator while that stream still uses them. */
    template <typename F>
    c10::intrusive_ptr<Work> run(c10d::OpType op, std::vector<at::Tensor> outputs, const at::Tensor& where, F fn, bool torch_ops = false,
                                 c10::intrusive_ptr<Work> after = nullptr, const std::vector<at::Tensor>& keep = {}) {
        std::lock_guard<std::mutex> g(mu_);
        TORCH_CHECK(comm_, "dccl backend: the process group was shut down");
        const bool cuda = where.is_cuda();
        auto work = c10::make_intrusive<WorkDccl>(op, std::move(outputs), cuda, comm_);
        if (!cuda) {
            check(fn(nullptr), "host collective");
            work->launched(nullptr);
            return work;
        }
        (void)after;   // same communication stream: already ordered
        if (coalescing_) coalesced_device_ = (int)where.device().index();
        c10::cuda::CUDAGuard dg(where.device());
        c10::cuda::CUDAStream& cs = comm_stream(where.device().index());
        at::cuda::CUDAEvent ready(cudaEventDisableTiming);
        ready.record(c10::cuda::getCurrentCUDAStream(where.device().index()));
        ready.block(cs);
        if (torch_ops) {
            c10::cuda::CUDAStreamGuard sg(cs);
            check(fn(cs.stream()), "device collective");
        } else {
            check(fn(cs.stream()), "device collective");
        }
        // tensors used on the communication stream must not be freed while it still runs
        for (auto& t : work->result()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cs);
        for (auto& t : keep) if (t.defined() && t.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cs);
        work->launched(&cs);
        return work;
    }

    dccl::ncclComm_t comm_ = nullptr;
    std::unique_ptr<c10::cuda::CUDAStream> stream_;
    std::mutex mu_;
    bool coalescing_ = false;
    int coalesced_device_ = -1;   // device of the CUDA tensors seen while coalescing, -1: host tensors only
};

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "PyTorch process-group backend of the DCCL B200 collective library";
    m.def("create_backend", &BackendDccl::create, "create a c10d backend over a store");
    m.def("comm_handle", [](const c10::intrusive_ptr<c10d::Backend>& b) -> uintptr_t {
        auto* d = dynamic_cast<BackendDccl*>(b.get());
        TORCH_CHECK(d, "not a dccl backend");
        return (uintptr_t)d->comm();
    }, "raw communicator handle (for dccl_b200.Communicator.from_handle)");
}
