// A c10d backend over the DICL communicator, for tensors on the "dipu" device of the eager adapter:
// torch.distributed.init_process_group("dicl") + dist.all_reduce(t) end in b200_dicl_all_reduce on a pool stream.
//
// It follows the structure of the reference's ProcessGroupDICL
// (dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:197-300 communicator set-up and unique-id exchange
// through the c10d store, :438-485 doComm, :71-193 WorkDICL): one device per process, the communicator created lazily on
// the first collective, rank 0's unique id published under a counter key of the store, collectives enqueued on a stream
// from the pool after it has waited for the producing stream, an event recorded behind them, and Work::wait() making the
// CURRENT stream wait for that event (no host block unless DICL_BLOCKING_WAIT=1). Tensors used on the communication stream
// are reported to the caching allocator (record_stream), as the reference does with dipu::recordStream.
// With DICL_BLOCKING_WAIT=1 the host polls the event and gives up with "Operation timed out!" after the time-out of the
// wait() call, or of the process group when the call names none (reference: WorkDICL::synchronize,
// ProcessGroupDICL.cpp:154-167, opTimeout_ at ProcessGroupDICL.h:40-41) - the path's failure detection for a peer that never
// arrives. gather / scatter are built from point-to-point transfers plus one device-to-device copy for the root's own part,
// the way the reference's proxy builds them (runtime/devproxy/diclproxy.cpp:61-105).
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include "../torch_adapter/adapter_common.h"

namespace dipu_b200 {
namespace {

#define DICL_CHECK(expr)                                                                                                \
    do {                                                                                                                \
        const b200Status_t st__ = (expr);                                                                               \
        TORCH_CHECK(st__ == B200_SUCCESS, #expr, " failed with status ", static_cast<int>(st__), ": ", b200_last_error()); \
    } while (0)

int to_dicl_op(const c10d::ReduceOp& op) {
    switch (op) {
        case c10d::ReduceOp::SUM: return B200_REDUCE_SUM;
        case c10d::ReduceOp::AVG: return B200_REDUCE_AVG;
        case c10d::ReduceOp::PRODUCT: return B200_REDUCE_PRODUCT;
        case c10d::ReduceOp::MIN: return B200_REDUCE_MIN;
        case c10d::ReduceOp::MAX: return B200_REDUCE_MAX;
        default: TORCH_CHECK(false, "dicl: reduce op ", static_cast<int>(static_cast<uint8_t>(op)), " is not supported");
    }
}

void check_tensor(const at::Tensor& t, const char* what) {
    TORCH_CHECK(t.device().type() == kDevice, "dicl: ", what, " must live on the dipu device, got ", t.device());
    TORCH_CHECK(t.is_contiguous(), "dicl: ", what, " must be contiguous");
}

// Host-side wait of the blocking mode: polls `done` until it holds, throws once `limit` has passed (0 = no limit).
template <typename Pred>
void blocking_wait(Pred done, std::chrono::milliseconds limit) {
    const auto t0 = std::chrono::steady_clock::now();
    while (!done()) {
        if (limit.count() > 0 && std::chrono::steady_clock::now() - t0 > limit) TORCH_CHECK(false, "Operation timed out!");
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

class WorkDICL final : public c10d::Work {
  public:
    WorkDICL(int rank, c10d::OpType op, int device, b200Comm_t comm, bool blocking, std::chrono::milliseconds op_timeout)
        : c10d::Work(rank, op), device_(device), comm_(comm), blocking_(blocking), op_timeout_(op_timeout) {
        DICL_CHECK(b200_event_from_pool(&event_));
    }
    ~WorkDICL() override {
        if (event_ != nullptr) (void)b200_event_to_pool(event_);
    }
    void record(b200Stream_t comm_stream) { DICL_CHECK(b200_record_event(event_, comm_stream)); }

    bool isCompleted() override {
        b200EventStatus_t st = B200_EVENT_READY;
        DICL_CHECK(b200_get_event_status(event_, &st));
        return st == B200_EVENT_READY;
    }
    bool isSuccess() const override { return b200_dicl_get_comm_async_error(comm_) == B200_SUCCESS; }
    // The stream the caller computes on waits for the collective; the host only blocks when asked to.
    bool wait(std::chrono::milliseconds timeout) override {
        DICL_CHECK(b200_stream_wait_event(current_stream(device_), event_));
        if (blocking_) blocking_wait([this] { return isCompleted(); }, timeout == kNoTimeout ? op_timeout_ : timeout);
        return true;
    }
    void synchronize() override { wait(std::chrono::milliseconds(0)); }
    std::vector<at::Tensor> result() override { return outputs_; }

    std::vector<at::Tensor> outputs_;  // keeps the results (and staging tensors) alive until the work is released

  private:
    int device_;
    b200Comm_t comm_;
    bool blocking_;
    std::chrono::milliseconds op_timeout_;
    b200Event_t event_ = nullptr;
};

class ProcessGroupDICL final : public c10d::Backend {
  public:
    ProcessGroupDICL(c10::intrusive_ptr<c10d::Store> store, int rank, int size, std::chrono::milliseconds op_timeout)
        : c10d::Backend(rank, size), store_(std::move(store)), op_timeout_(op_timeout) {
        const char* b = std::getenv("DICL_BLOCKING_WAIT");
        blocking_ = b != nullptr && std::strcmp(b, "1") == 0;
    }
    ~ProcessGroupDICL() override {
        if (comm_ != nullptr) {
            (void)b200_sync_stream(comm_stream_);
            (void)b200_dicl_comm_destroy(comm_);
        }
    }
    const std::string getBackendName() const override { return "dicl"; }

    c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "dicl: one tensor per call (one device per process)");
        at::Tensor& t = tensors[0];
        check_tensor(t, "all_reduce tensor");
        const int op = to_dicl_op(opts.reduceOp);
        return run(c10d::OpType::ALLREDUCE, {t}, {t}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_all_reduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), to_diopi_dtype(t.scalar_type()), op, comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "dicl: one tensor per call");
        at::Tensor& t = tensors[0];
        check_tensor(t, "broadcast tensor");
        const int root = static_cast<int>(opts.rootRank);
        return run(c10d::OpType::BROADCAST, {t}, {t}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_broadcast(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), to_diopi_dtype(t.scalar_type()), root, comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "dicl: one tensor per call");
        at::Tensor& t = tensors[0];
        check_tensor(t, "reduce tensor");
        const int op = to_dicl_op(opts.reduceOp), root = static_cast<int>(opts.rootRank);
        return run(c10d::OpType::REDUCE, {t}, {t}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_reduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), to_diopi_dtype(t.scalar_type()), op, root, comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input, const c10d::AllgatherOptions&) override {
        check_tensor(output, "all_gather output");
        check_tensor(input, "all_gather input");
        TORCH_CHECK(output.numel() == input.numel() * getSize() && output.scalar_type() == input.scalar_type(),
                    "dicl: all_gather output must hold world_size inputs of the same dtype");
        return run(c10d::OpType::_ALLGATHER_BASE, {input}, {output}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_all_gather(input.data_ptr(), output.data_ptr(), static_cast<size_t>(input.numel()), to_diopi_dtype(input.scalar_type()), comm, s));
        });
    }

    // list form: gathered into one flat tensor on the communication stream, then copied out on the current stream
    c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                             const c10d::AllgatherOptions& opts) override {
        TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1 && static_cast<int>(outputs[0].size()) == getSize(),
                    "dicl: all_gather expects one input and world_size outputs");
        at::Tensor input = inputs[0];
        check_tensor(input, "all_gather input");
        at::Tensor flat = at::empty({getSize(), input.numel()}, input.options());
        auto work = _allgather_base(flat, input, opts);
        work->wait();  // stream-level: the copies below are ordered behind the collective
        for (int r = 0; r < getSize(); ++r) outputs[0][r].copy_(flat[r].view_as(outputs[0][r]));
        return work;
    }

    c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) override {
        check_tensor(output, "reduce_scatter output");
        check_tensor(input, "reduce_scatter input");
        TORCH_CHECK(input.numel() == output.numel() * getSize() && output.scalar_type() == input.scalar_type(),
                    "dicl: reduce_scatter input must hold world_size outputs of the same dtype");
        const int op = to_dicl_op(opts.reduceOp);
        return run(c10d::OpType::_REDUCE_SCATTER_BASE, {input}, {output}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_reduce_scatter(input.data_ptr(), output.data_ptr(), static_cast<size_t>(output.numel()),
                                                to_diopi_dtype(input.scalar_type()), op, comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& out_splits, std::vector<int64_t>& in_splits,
                                                 const c10d::AllToAllOptions&) override {
        check_tensor(output, "all_to_all output");
        check_tensor(input, "all_to_all input");
        TORCH_CHECK(out_splits.empty() && in_splits.empty(), "dicl: all_to_all_single with explicit splits is not supported through this backend");
        TORCH_CHECK(input.numel() == output.numel() && input.numel() % getSize() == 0, "dicl: all_to_all tensors must divide evenly by world_size");
        return run(c10d::OpType::ALLTOALL_BASE, {input}, {output}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_all_to_all_equal_split(input.data_ptr(), output.data_ptr(), static_cast<size_t>(input.numel() / getSize()),
                                                        to_diopi_dtype(input.scalar_type()), comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int /*tag*/) override {
        TORCH_CHECK(tensors.size() == 1, "dicl: one tensor per call");
        at::Tensor& t = tensors[0];
        check_tensor(t, "send tensor");
        return run(c10d::OpType::SEND, {t}, {}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_send(t.data_ptr(), static_cast<size_t>(t.numel()), to_diopi_dtype(t.scalar_type()), dst, comm, s));
        });
    }

    c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int /*tag*/) override {
        TORCH_CHECK(tensors.size() == 1, "dicl: one tensor per call");
        at::Tensor& t = tensors[0];
        check_tensor(t, "recv tensor");
        return run(c10d::OpType::RECV, {}, {t}, [&](b200Comm_t comm, b200Stream_t s) {
            DICL_CHECK(b200_dicl_recv(t.data_ptr(), static_cast<size_t>(t.numel()), to_diopi_dtype(t.scalar_type()), src, comm, s));
        });
    }

    // root receives one part from every other rank and copies its own part; the others send theirs
    c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                          const c10d::GatherOptions& opts) override {
        TORCH_CHECK(inputs.size() == 1, "dicl: gather expects one input tensor");
        at::Tensor input = inputs[0];
        check_tensor(input, "gather input");
        const int root = static_cast<int>(opts.rootRank), me = getRank(), n = getSize();
        std::vector<at::Tensor> outs;
        if (me == root) {
            TORCH_CHECK(outputs.size() == 1 && static_cast<int>(outputs[0].size()) == n, "dicl: gather expects world_size outputs on the root");
            outs = outputs[0];
            for (const at::Tensor& o : outs) {
                check_tensor(o, "gather output");
                TORCH_CHECK(o.numel() == input.numel() && o.scalar_type() == input.scalar_type(), "dicl: gather outputs must match the input");
            }
        } else {
            TORCH_CHECK(outputs.empty() || outputs[0].empty(), "dicl: gather outputs are only given on the root");
        }
        const size_t count = static_cast<size_t>(input.numel());
        const int dt = to_diopi_dtype(input.scalar_type());
        return run(c10d::OpType::GATHER, {input}, outs, [&](b200Comm_t comm, b200Stream_t s) {
            if (me != root) {
                DICL_CHECK(b200_dicl_send(input.data_ptr(), count, dt, root, comm, s));
                return;
            }
            const int dev = input.device().index();
            for (int r = 0; r < n; ++r) {
                if (r == root) DICL_CHECK(b200_memcpy_d2d_async(s, count * input.element_size(), dev, outs[r].data_ptr(), dev, input.data_ptr()));
                else DICL_CHECK(b200_dicl_recv(outs[r].data_ptr(), count, dt, r, comm, s));
            }
        });
    }

    // root sends one part to every other rank and copies its own part; the others receive theirs
    c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                           const c10d::ScatterOptions& opts) override {
        TORCH_CHECK(outputs.size() == 1, "dicl: scatter expects one output tensor");
        at::Tensor output = outputs[0];
        check_tensor(output, "scatter output");
        const int root = static_cast<int>(opts.rootRank), me = getRank(), n = getSize();
        std::vector<at::Tensor> ins;
        if (me == root) {
            TORCH_CHECK(inputs.size() == 1 && static_cast<int>(inputs[0].size()) == n, "dicl: scatter expects world_size inputs on the root");
            ins = inputs[0];
            for (const at::Tensor& t : ins) {
                check_tensor(t, "scatter input");
                TORCH_CHECK(t.numel() == output.numel() && t.scalar_type() == output.scalar_type(), "dicl: scatter inputs must match the output");
            }
        } else {
            TORCH_CHECK(inputs.empty() || inputs[0].empty(), "dicl: scatter inputs are only given on the root");
        }
        const size_t count = static_cast<size_t>(output.numel());
        const int dt = to_diopi_dtype(output.scalar_type());
        return run(c10d::OpType::SCATTER, ins, {output}, [&](b200Comm_t comm, b200Stream_t s) {
            if (me != root) {
                DICL_CHECK(b200_dicl_recv(output.data_ptr(), count, dt, root, comm, s));
                return;
            }
            const int dev = output.device().index();
            for (int r = 0; r < n; ++r) {
                if (r == root) DICL_CHECK(b200_memcpy_d2d_async(s, count * output.element_size(), dev, output.data_ptr(), dev, ins[r].data_ptr()));
                else DICL_CHECK(b200_dicl_send(ins[r].data_ptr(), count, dt, r, comm, s));
            }
        });
    }

    c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions&) override {
        int dev = 0;
        DICL_CHECK(b200_current_device(&dev));
        at::Tensor token = at::zeros({1}, at::TensorOptions().dtype(at::kFloat).device(c10::Device(kDevice, static_cast<c10::DeviceIndex>(dev))));
        std::vector<at::Tensor> v{token};
        auto work = allreduce(v, c10d::AllreduceOptions());
        work->wait();
        DICL_CHECK(b200_sync_stream(current_stream(dev)));  // a barrier is a host-level rendezvous
        return work;
    }

  private:
    // The communicator of this process: created on first use on the device of the tensors, unique id from rank 0 through
    // the store under a per-communicator key.
    void ensure_comm(int device) {
        std::lock_guard<std::mutex> lock(mu_);
        if (comm_ != nullptr) {
            TORCH_CHECK(device == device_, "dicl: one device per process; the communicator lives on dipu:", device_, ", got dipu:", device);
            return;
        }
        DICL_CHECK(b200_set_device(device));
        b200UniqueId id;
        std::memset(&id, 0, sizeof(id));
        const std::string key = "dicl_unique_id_" + std::to_string(comm_counter_++);
        if (getRank() == 0) {
            DICL_CHECK(b200_dicl_get_unique_id(&id));
            const auto* bytes = reinterpret_cast<const uint8_t*>(&id);
            store_->set(key, std::vector<uint8_t>(bytes, bytes + sizeof(id)));
        } else {
            const std::vector<uint8_t> bytes = store_->get(key);
            TORCH_CHECK(bytes.size() == sizeof(id), "dicl: unexpected unique-id length in the store: ", bytes.size());
            std::memcpy(&id, bytes.data(), sizeof(id));
        }
        DICL_CHECK(b200_stream_from_pool(device, &comm_stream_));
        DICL_CHECK(b200_dicl_comm_init_rank(&comm_, getSize(), &id, getRank(), device));
        device_ = device;
    }

    template <typename Fn>
    c10::intrusive_ptr<c10d::Work> run(c10d::OpType op, std::vector<at::Tensor> inputs, std::vector<at::Tensor> outputs, Fn fn) {
        const at::Tensor& any = !inputs.empty() ? inputs[0] : outputs[0];
        const int device = any.device().index();
        ensure_comm(device);
        const c10::DeviceGuard guard(any.device());
        // the communication stream first waits for what the compute stream has enqueued so far
        b200Event_t pre = nullptr;
        DICL_CHECK(b200_event_from_pool(&pre));
        DICL_CHECK(b200_record_event(pre, current_stream(device)));
        DICL_CHECK(b200_stream_wait_event(comm_stream_, pre));
        DICL_CHECK(b200_event_to_pool(pre));
        auto work = c10::make_intrusive<WorkDICL>(getRank(), op, device, comm_, blocking_, op_timeout_);
        fn(comm_, comm_stream_);
        for (const auto* list : {&inputs, &outputs}) {
            for (const at::Tensor& t : *list) {
                if (t.has_storage() && t.storage().data() != nullptr) (void)b200_cache_record_stream(t.storage().mutable_data(), comm_stream_);
            }
        }
        work->record(comm_stream_);
        work->outputs_ = std::move(outputs);
        return work;
    }

    c10::intrusive_ptr<c10d::Store> store_;
    std::mutex mu_;
    b200Comm_t comm_ = nullptr;
    b200Stream_t comm_stream_ = nullptr;
    int device_ = -1;
    int comm_counter_ = 0;
    bool blocking_ = false;
    std::chrono::milliseconds op_timeout_;
};

c10::intrusive_ptr<c10d::Backend> create_process_group_dicl(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                            const std::chrono::duration<float>& timeout) {
    return c10::make_intrusive<ProcessGroupDICL>(store, rank, size, std::chrono::duration_cast<std::chrono::milliseconds>(timeout));
}

// Host-only exercise of the blocking wait: a condition that becomes true after `ready_after_ms` (never, when negative),
// waited for with a limit of `timeout_ms`. Returns the milliseconds waited; throws "Operation timed out!" like Work::wait.
double blocking_wait_selftest(int64_t timeout_ms, int64_t ready_after_ms) {
    const auto t0 = std::chrono::steady_clock::now();
    blocking_wait(
        [&] {
            if (ready_after_ms < 0) return false;
            return std::chrono::steady_clock::now() - t0 >= std::chrono::milliseconds(ready_after_ms);
        },
        std::chrono::milliseconds(timeout_ms));
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

}  // namespace
}  // namespace dipu_b200

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "c10d backend 'dicl' over the B200 DICL communicator";
    m.def("create_process_group_dicl", &dipu_b200::create_process_group_dicl, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"));
    m.def("blocking_wait_selftest", &dipu_b200::blocking_wait_selftest, py::arg("timeout_ms"), py::arg("ready_after_ms"));
}
