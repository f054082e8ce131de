// promethorch C++ API: process groups, DistributedDataParallel with no_sync, tensor-parallel linear layers, a
// fork-based launcher and DistributedSampler (names of torch/distributed/ddp.h:37-186, distributed.h, launcher.h,
// torch/nn/parallel/tensor_parallel.h:72-554 and torch/data/distributed_sampler.h of the reference).
//
// The C++ process group is the CPU/TCP plumbing path (rank 0 is the hub: length-prefixed messages over loopback or
// Ethernet, receive/send timeouts), which is what the reference's C++ programs use and what needs no GPU.  On GPUs the
// framework's collectives are the fused peer-memory kernels of libptb200 driven from the Python package; a CUDA tensor
// handed to this group is staged through the host.
#pragma once
#include <torch/torch.h>

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <functional>
#include <memory>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace promethorch {
using Tensor = at::Tensor;

namespace distributed {

struct DDPConfig {
    int rank = 0;
    int world_size = 1;
    std::string master_addr = "127.0.0.1";
    int master_port = 29500;
    int timeout_sec = 300;
};

enum class ReduceOp { SUM, AVG, MAX, MIN };
enum class BackendType { TCP, SINGLE };

struct CollectiveTimeout : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class ProcessGroup {
 public:
    virtual ~ProcessGroup() = default;
    virtual int rank() const = 0;
    virtual int world_size() const = 0;
    virtual void all_reduce(Tensor& t, ReduceOp op = ReduceOp::SUM) = 0;
    virtual void broadcast(Tensor& t, int src = 0) = 0;
    virtual void barrier() = 0;
    // out[r] = rank r's `t` (all the same shape)
    virtual std::vector<Tensor> all_gather(const Tensor& t) = 0;
};
using ProcessGroupPtr = std::shared_ptr<ProcessGroup>;

class SingleProcessGroup : public ProcessGroup {
 public:
    int rank() const override { return 0; }
    int world_size() const override { return 1; }
    void all_reduce(Tensor&, ReduceOp) override {}
    void broadcast(Tensor&, int) override {}
    void barrier() override {}
    std::vector<Tensor> all_gather(const Tensor& t) override { return {t.clone()}; }
};

// Counts calls and moves nothing: the fake the no_sync tests use (world size 2, as in tests/test_ddp_no_sync.cpp).
class CountingPG : public ProcessGroup {
 public:
    CountingPG(int rank = 0, int world = 2) : rank_(rank), world_(world) {}
    int rank() const override { return rank_; }
    int world_size() const override { return world_; }
    void all_reduce(Tensor&, ReduceOp) override { ++all_reduce_calls; }
    void broadcast(Tensor&, int) override { ++broadcast_calls; }
    void barrier() override { ++barrier_calls; }
    std::vector<Tensor> all_gather(const Tensor& t) override { return std::vector<Tensor>(world_, t.clone()); }
    int all_reduce_calls = 0, broadcast_calls = 0, barrier_calls = 0;

 private:
    int rank_, world_;
};

// Rank 0 listens, the others connect; every message is an 8-byte length followed by the payload.
class TCPProcessGroup : public ProcessGroup {
 public:
    explicit TCPProcessGroup(const DDPConfig& c) : cfg_(c) {
        if (c.world_size <= 1) return;
        if (c.rank == 0) {
            const int ls = ::socket(AF_INET, SOCK_STREAM, 0);
            check(ls >= 0, "socket");
            int one = 1;
            ::setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
            sockaddr_in a{};
            a.sin_family = AF_INET;
            a.sin_addr.s_addr = htonl(INADDR_ANY);
            a.sin_port = htons((uint16_t)c.master_port);
            check(::bind(ls, (sockaddr*)&a, sizeof(a)) == 0, "bind");
            check(::listen(ls, c.world_size) == 0, "listen");
            set_timeouts(ls);
            peers_.assign(c.world_size, -1);
            for (int k = 1; k < c.world_size; ++k) {
                const int fd = ::accept(ls, nullptr, nullptr);
                if (fd < 0) { ::close(ls); throw CollectiveTimeout("rendezvous: a rank did not connect within the timeout"); }
                set_timeouts(fd);
                int32_t r = -1;
                recv_all(fd, &r, sizeof(r));
                check(r > 0 && r < c.world_size && peers_[r] < 0, "rank handshake");
                peers_[r] = fd;
                const char ack = 1;
                send_all(fd, &ack, 1);
            }
            ::close(ls);
        } else {
            sockaddr_in a{};
            a.sin_family = AF_INET;
            a.sin_port = htons((uint16_t)c.master_port);
            check(::inet_pton(AF_INET, c.master_addr.c_str(), &a.sin_addr) == 1, "master address");
            const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(c.timeout_sec);
            for (;;) {
                hub_ = ::socket(AF_INET, SOCK_STREAM, 0);
                check(hub_ >= 0, "socket");
                if (::connect(hub_, (sockaddr*)&a, sizeof(a)) == 0) break;
                ::close(hub_);
                hub_ = -1;
                if (std::chrono::steady_clock::now() > deadline) throw CollectiveTimeout("rendezvous: rank 0 is not listening");
                std::this_thread::sleep_for(std::chrono::milliseconds(20));
            }
            set_timeouts(hub_);
            const int32_t r = c.rank;
            send_all(hub_, &r, sizeof(r));
            char ack = 0;
            recv_all(hub_, &ack, 1);
        }
    }
    ~TCPProcessGroup() override {
        for (int fd : peers_) if (fd >= 0) ::close(fd);
        if (hub_ >= 0) ::close(hub_);
    }
    int rank() const override { return cfg_.rank; }
    int world_size() const override { return cfg_.world_size; }

    void all_reduce(Tensor& t, ReduceOp op = ReduceOp::SUM) override {
        if (cfg_.world_size <= 1) return;
        Tensor h = t.detach().to(torch::kCPU, torch::kFloat).contiguous();
        if (cfg_.rank == 0) {
            Tensor tmp = torch::empty_like(h);
            for (int r = 1; r < cfg_.world_size; ++r) {
                recv_msg(peers_[r], tmp.data_ptr(), (size_t)tmp.numel() * 4);
                if (op == ReduceOp::MAX) h = torch::maximum(h, tmp);
                else if (op == ReduceOp::MIN) h = torch::minimum(h, tmp);
                else h.add_(tmp);
            }
            if (op == ReduceOp::AVG) h.div_((double)cfg_.world_size);
            for (int r = 1; r < cfg_.world_size; ++r) send_msg(peers_[r], h.data_ptr(), (size_t)h.numel() * 4);
        } else {
            send_msg(hub_, h.data_ptr(), (size_t)h.numel() * 4);
            recv_msg(hub_, h.data_ptr(), (size_t)h.numel() * 4);
        }
        torch::NoGradGuard ng;
        t.copy_(h.to(t.dtype()).view_as(t));
    }
    void broadcast(Tensor& t, int src = 0) override {
        if (cfg_.world_size <= 1) return;
        Tensor h = t.detach().to(torch::kCPU).contiguous();
        const size_t n = (size_t)h.numel() * h.element_size();
        if (cfg_.rank == 0) {
            if (src != 0) recv_msg(peers_[src], h.data_ptr(), n);
            for (int r = 1; r < cfg_.world_size; ++r)
                if (r != src) send_msg(peers_[r], h.data_ptr(), n);
        } else if (cfg_.rank == src) {
            send_msg(hub_, h.data_ptr(), n);
        } else {
            recv_msg(hub_, h.data_ptr(), n);
        }
        torch::NoGradGuard ng;
        t.copy_(h.view_as(t));
    }
    void barrier() override {
        Tensor z = torch::zeros({1});
        all_reduce(z, ReduceOp::SUM);
    }
    std::vector<Tensor> all_gather(const Tensor& t) override {
        Tensor h = t.detach().to(torch::kCPU).contiguous();
        const int W = cfg_.world_size;
        std::vector<Tensor> out;
        if (W <= 1) return {h.clone()};
        const size_t n = (size_t)h.numel() * h.element_size();
        Tensor all = torch::empty({W, h.numel()}, h.options());
        if (cfg_.rank == 0) {
            all[0].copy_(h.view(-1));
            for (int r = 1; r < W; ++r) recv_msg(peers_[r], all[r].data_ptr(), n);
            for (int r = 1; r < W; ++r) send_msg(peers_[r], all.data_ptr(), n * W);
        } else {
            send_msg(hub_, h.data_ptr(), n);
            recv_msg(hub_, all.data_ptr(), n * W);
        }
        for (int r = 0; r < W; ++r) out.push_back(all[r].view_as(h).clone());
        return out;
    }

 private:
    static void check(bool ok, const char* what) {
        if (!ok) throw std::runtime_error(std::string("TCP process group: ") + what + " failed: " + std::strerror(errno));
    }
    void set_timeouts(int fd) const {
        timeval tv{cfg_.timeout_sec, 0};
        ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
        int one = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    }
    static void send_all(int fd, const void* p, size_t n) {
        const char* c = (const char*)p;
        while (n) {
            const ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
            if (k <= 0) throw CollectiveTimeout("send failed or timed out: the peer is gone or too far behind");
            c += k;
            n -= (size_t)k;
        }
    }
    static void recv_all(int fd, void* p, size_t n) {
        char* c = (char*)p;
        while (n) {
            const ssize_t k = ::recv(fd, c, n, 0);
            if (k <= 0) throw CollectiveTimeout("receive failed or timed out: the peer is gone or too far behind");
            c += k;
            n -= (size_t)k;
        }
    }
    static void send_msg(int fd, const void* p, size_t n) {
        const uint64_t len = n;
        send_all(fd, &len, sizeof(len));
        send_all(fd, p, n);
    }
    static void recv_msg(int fd, void* p, size_t n) {
        uint64_t len = 0;
        recv_all(fd, &len, sizeof(len));
        if (len != n) throw std::runtime_error("TCP process group: message of " + std::to_string(len) + " bytes, expected " + std::to_string(n));
        recv_all(fd, p, n);
    }
    DDPConfig cfg_;
    std::vector<int> peers_;
    int hub_ = -1;
};

// ---- the default (process-wide) group
inline ProcessGroupPtr& default_group() {
    static ProcessGroupPtr g;
    return g;
}
inline void init_process_group(const DDPConfig& cfg) {
    default_group() = cfg.world_size > 1 ? ProcessGroupPtr(new TCPProcessGroup(cfg)) : ProcessGroupPtr(new SingleProcessGroup());
}
inline void destroy_process_group() { default_group().reset(); }
inline bool is_initialized() { return (bool)default_group(); }
inline int get_rank() { return default_group() ? default_group()->rank() : 0; }
inline int get_world_size() { return default_group() ? default_group()->world_size() : 1; }
inline void all_reduce(Tensor& t, ReduceOp op = ReduceOp::SUM) { if (default_group()) default_group()->all_reduce(t, op); }
inline void all_reduce_inplace(float* p, int64_t n) {
    Tensor t = torch::from_blob(p, {n}, torch::kFloat);
    all_reduce(t);
}
inline void broadcast(Tensor& t, int src = 0) { if (default_group()) default_group()->broadcast(t, src); }
inline void barrier() { if (default_group()) default_group()->barrier(); }
inline void init_process_group_single_rank() { default_group() = ProcessGroupPtr(new SingleProcessGroup()); }
// buf holds world_size slices of `per_rank` floats; this rank's slice is filled in, the others are received.
inline void all_gather_inplace(float* buf, int64_t per_rank) {
    if (!default_group() || default_group()->world_size() <= 1) return;
    const int r = default_group()->rank();
    Tensor mine = torch::from_blob(buf + (int64_t)r * per_rank, {per_rank}, torch::kFloat).clone();
    auto parts = default_group()->all_gather(mine);
    for (size_t k = 0; k < parts.size(); ++k) std::memcpy(buf + (int64_t)k * per_rank, parts[k].data_ptr(), sizeof(float) * (size_t)per_rank);
}
// Split form: post starts the gather on a helper thread, wait joins it (overlap with independent work in between; no
// other collective of the same group may run until wait returns).
struct AllGatherHandle {
    std::shared_ptr<std::thread> worker;
    std::shared_ptr<std::exception_ptr> error;
};
inline AllGatherHandle all_gather_post(float* buf, int64_t per_rank) {
    AllGatherHandle h;
    h.error = std::make_shared<std::exception_ptr>();
    auto err = h.error;
    h.worker = std::make_shared<std::thread>([buf, per_rank, err] {
        try { all_gather_inplace(buf, per_rank); } catch (...) { *err = std::current_exception(); }
    });
    return h;
}
inline void all_gather_wait(AllGatherHandle& h) {
    if (h.worker && h.worker->joinable()) h.worker->join();
    if (h.error && *h.error) std::rethrow_exception(*h.error);
}

// DistributedDataParallel: parameters and buffers are broadcast from rank 0 at construction; after backward,
// allreduce_grads() (alias finish_gradient_synchronization / sync_gradients) averages every gradient over the ranks,
// unless gradient synchronisation is switched off (DDPNoSyncGuard), in which case gradients keep accumulating locally.
template <typename ModuleHolder>
class DistributedDataParallel {
 public:
    explicit DistributedDataParallel(ModuleHolder module, ProcessGroupPtr pg = nullptr, bool broadcast_parameters = true)
        : module_(std::move(module)), pg_(pg ? pg : (default_group() ? default_group() : ProcessGroupPtr(new SingleProcessGroup()))) {
        if (broadcast_parameters && pg_->world_size() > 1) {
            torch::NoGradGuard ng;
            for (auto& p : module_->parameters()) pg_->broadcast(p, 0);
            for (auto& b : module_->buffers()) pg_->broadcast(b, 0);
        }
    }
    template <typename... Args>
    auto forward(Args&&... args) { return module_->forward(std::forward<Args>(args)...); }
    template <typename... Args>
    auto operator()(Args&&... args) { return forward(std::forward<Args>(args)...); }
    void allreduce_grads() {
        if (!require_grad_sync_ || pg_->world_size() <= 1) return;
        for (auto& p : module_->parameters())
            if (p.grad().defined()) pg_->all_reduce(p.mutable_grad(), ReduceOp::AVG);
    }
    void finish_gradient_synchronization() { allreduce_grads(); }
    void sync_gradients() {
        const bool keep = require_grad_sync_;
        require_grad_sync_ = true;
        allreduce_grads();
        require_grad_sync_ = keep;
    }
    bool require_grad_sync() const { return require_grad_sync_; }
    void set_require_grad_sync(bool v) { require_grad_sync_ = v; }
    ModuleHolder& module() { return module_; }
    int rank() const { return pg_->rank(); }
    int world_size() const { return pg_->world_size(); }
    ProcessGroupPtr process_group() const { return pg_; }

 private:
    ModuleHolder module_;
    ProcessGroupPtr pg_;
    bool require_grad_sync_ = true;
};

// Scope in which gradient synchronisation is off; restores the previous setting, nests, cannot be copied.
template <typename DDP>
class DDPNoSyncGuard {
 public:
    explicit DDPNoSyncGuard(DDP& ddp) : ddp_(ddp), prev_(ddp.require_grad_sync()) { ddp_.set_require_grad_sync(false); }
    ~DDPNoSyncGuard() { ddp_.set_require_grad_sync(prev_); }
    DDPNoSyncGuard(const DDPNoSyncGuard&) = delete;
    DDPNoSyncGuard& operator=(const DDPNoSyncGuard&) = delete;

 private:
    DDP& ddp_;
    bool prev_;
};

// Fork `world_size` processes that run fn(rank, config); returns the worst exit code (128 + signal for a killed rank).
// Call it before the calling process has run tensor operations: those start libtorch's worker threads, and a child
// forked from a multi-threaded process inherits their locks without the threads.
struct DistArgs {
    int rank = 0, world_size = 1;
    std::string master_addr = "127.0.0.1";
    int master_port = 29500;
};
inline int launch(int world_size, const std::function<int(const DistArgs&)>& fn, const std::string& addr = "127.0.0.1", int port = 29500) {
    std::vector<pid_t> kids;
    for (int r = 0; r < world_size; ++r) {
        const pid_t pid = ::fork();
        if (pid < 0) {
            for (pid_t k : kids) ::kill(k, SIGTERM);       // exactly the children started here
            throw std::runtime_error("launch: fork failed");
        }
        if (pid == 0) {
            DistArgs a{r, world_size, addr, port};
            ::setenv("RANK", std::to_string(r).c_str(), 1);
            ::setenv("WORLD_SIZE", std::to_string(world_size).c_str(), 1);
            ::setenv("MASTER_ADDR", addr.c_str(), 1);
            ::setenv("MASTER_PORT", std::to_string(port).c_str(), 1);
            int rc = 1;
            try { rc = fn(a); } catch (const std::exception& e) { std::fprintf(stderr, "[rank %d] %s\n", r, e.what()); }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    int worst = 0;
    for (pid_t k : kids) {
        int st = 0;
        ::waitpid(k, &st, 0);
        const int rc = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + WTERMSIG(st);
        worst = std::max(worst, rc);
    }
    return worst;
}
inline DistArgs parse_dist_args(int argc, char** argv) {
    DistArgs a;
    for (int i = 1; i + 1 < argc; ++i) {
        const std::string k = argv[i];
        if (k == "--rank") a.rank = std::atoi(argv[++i]);
        else if (k == "--world-size" || k == "--world_size" || k == "--nprocs") a.world_size = std::atoi(argv[++i]);
        else if (k == "--master-addr" || k == "--master_addr") a.master_addr = argv[++i];
        else if (k == "--master-port" || k == "--master_port") a.master_port = std::atoi(argv[++i]);
    }
    return a;
}

}  // namespace distributed

namespace data {
// The indices of one rank: shuffle with seed + epoch, pad (or drop) to a multiple of the world size, take
// indices[rank::world] (the rule of torch.utils.data.DistributedSampler).
class DistributedSampler {
 public:
    DistributedSampler(int64_t dataset_size, int world_size, int rank, bool shuffle = true, uint64_t seed = 0, bool drop_last = false)
        : n_(dataset_size), world_(world_size), rank_(rank), shuffle_(shuffle), seed_(seed), drop_last_(drop_last) {}
    void set_epoch(int64_t e) { epoch_ = e; }
    int64_t num_samples() const { return drop_last_ ? n_ / world_ : (n_ + world_ - 1) / world_; }
    std::vector<int64_t> indices() const {
        std::vector<int64_t> idx(n_);
        std::iota(idx.begin(), idx.end(), 0);
        if (shuffle_) {
            std::mt19937_64 gen(seed_ + (uint64_t)epoch_);
            std::shuffle(idx.begin(), idx.end(), gen);
        }
        const int64_t total = num_samples() * world_;
        if (drop_last_) idx.resize(total);
        else for (int64_t i = 0; (int64_t)idx.size() < total; ++i) idx.push_back(idx[i]);
        std::vector<int64_t> mine;
        for (int64_t i = rank_; i < total; i += world_) mine.push_back(idx[i]);
        return mine;
    }

 private:
    int64_t n_;
    int world_, rank_;
    bool shuffle_;
    uint64_t seed_;
    bool drop_last_;
    int64_t epoch_ = 0;
};
}  // namespace data

namespace nn {
namespace parallel {

struct TPConfig {
    int rank = 0;
    int world_size = 1;
    distributed::ProcessGroupPtr pg;          // default: the process-wide group
    distributed::ProcessGroupPtr group() const { return pg ? pg : distributed::default_group(); }
};

inline Tensor tp_all_gather(const Tensor& local, const TPConfig& tp) {        // concatenates along the last dimension
    if (tp.world_size <= 1) return local;
    auto parts = tp.group()->all_gather(local);
    for (auto& p : parts) p = p.to(local.device());
    parts[tp.rank] = local;                      // the local slice keeps its autograd history (backward of a gather is a split)
    return torch::cat(parts, -1);
}
inline Tensor tp_all_reduce_sum(const Tensor& t, const TPConfig& tp) {
    if (tp.world_size <= 1) return t;
    Tensor out = t.clone();
    tp.group()->all_reduce(out, distributed::ReduceOp::SUM);
    return out;
}
inline void tp_barrier(const TPConfig& tp) { if (tp.world_size > 1) tp.group()->barrier(); }

// The full weight is drawn from a seeded generator on every rank and sliced, so a sharded layer computes exactly what
// the unsharded layer with the same seed computes.
inline Tensor tp_full_weight(int64_t out, int64_t in, uint64_t seed) {
    auto gen = at::detail::createCPUGenerator(seed);
    const double bound = 1.0 / std::sqrt((double)in);
    return torch::empty({out, in}).uniform_(-bound, bound, gen);
}

// y = x W^T with W[out, in] split by rows: every rank holds out/world rows; gather_output concatenates the outputs.
class ColumnParallelLinearImpl : public torch::nn::Module {
 public:
    ColumnParallelLinearImpl(int64_t in, int64_t out, TPConfig tp, bool gather_output = true, bool bias = true, uint64_t init_seed = 42)
        : tp_(std::move(tp)), gather_(gather_output) {
        TORCH_CHECK(out % tp_.world_size == 0, "ColumnParallelLinear: out_features must divide by the world size");
        const int64_t per = out / tp_.world_size;
        weight = register_parameter("weight", tp_full_weight(out, in, init_seed).narrow(0, tp_.rank * per, per).clone());
        if (bias) this->bias = register_parameter("bias", torch::zeros({per}));
    }
    Tensor forward(const Tensor& x) {
        Tensor y = torch::nn::functional::linear(x, weight, bias);
        return gather_ ? tp_all_gather(y, tp_) : y;
    }
    Tensor weight, bias;

 private:
    TPConfig tp_;
    bool gather_;
};
TORCH_MODULE(ColumnParallelLinear);

// y = x W^T with W[out, in] split by columns: every rank multiplies its slice of the input, the partial outputs are
// summed over the ranks, the bias is added once.
class RowParallelLinearImpl : public torch::nn::Module {
 public:
    RowParallelLinearImpl(int64_t in, int64_t out, TPConfig tp, bool input_is_parallel = true, bool bias = true, uint64_t init_seed = 42)
        : tp_(std::move(tp)), parallel_in_(input_is_parallel) {
        TORCH_CHECK(in % tp_.world_size == 0, "RowParallelLinear: in_features must divide by the world size");
        per_ = in / tp_.world_size;
        weight = register_parameter("weight", tp_full_weight(out, in, init_seed).narrow(1, tp_.rank * per_, per_).clone());
        if (bias) this->bias = register_parameter("bias", torch::zeros({out}));
    }
    Tensor forward(const Tensor& x) {
        Tensor xl = parallel_in_ ? x : x.narrow(-1, tp_.rank * per_, per_);
        Tensor y = tp_all_reduce_sum(torch::matmul(xl, weight.t()), tp_);
        return bias.defined() ? y + bias : y;
    }
    Tensor weight, bias;

 private:
    TPConfig tp_;
    bool parallel_in_;
    int64_t per_ = 0;
};
TORCH_MODULE(RowParallelLinear);

}  // namespace parallel
}  // namespace nn
}  // namespace promethorch
