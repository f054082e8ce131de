// promethorch C++ API: pipeline parallelism.
//
//  * Pipeline: GPipe inside one process.  The stages run in order over `chunks` micro-batches cut along dimension 0;
//    autograd carries the backward pass, gradients accumulate over the micro-batches
//    (torch/nn/parallel/pipeline.h of the reference).
//  * Pipeline1F1BStage: one stage of a pipeline whose stages are separate processes, scheduled one-forward-one-backward:
//    stage s runs S - s - 1 warm-up forwards, then alternates a forward with a backward, then drains the backwards,
//    so at most S - s micro-batches of activations are alive (torch/distributed/pipeline_schedule.h:60-260;
//    PipelineScheduleConfig{num_stages, num_micros, sync_dir, timeout_ms, poll_us}).  The reference passes activations
//    through files in sync_dir; here neighbouring stages talk over one TCP connection each (stage s listens on
//    base_port + s), sends are queued to a sender thread so that two neighbours sending at the same time cannot block
//    each other, and every receive is bounded by timeout_ms.
#pragma once
#include <torch/torch.h>

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "distributed.h"

namespace promethorch {
namespace nn {
namespace parallel {
using Tensor = at::Tensor;

class Pipeline {
 public:
    using Stage = std::function<Tensor(const Tensor&)>;
    Pipeline(std::vector<Stage> stages, int64_t chunks) : stages_(std::move(stages)), chunks_(chunks) {
        TORCH_CHECK(chunks_ >= 1 && !stages_.empty(), "Pipeline: at least one stage and one chunk");
    }
    // Sequential modules as stages.
    static Pipeline from_modules(std::vector<torch::nn::Sequential> mods, int64_t chunks) {
        std::vector<Stage> st;
        for (auto& m : mods) st.push_back([m](const Tensor& x) mutable { return m->forward(x); });
        return Pipeline(std::move(st), chunks);
    }
    Tensor forward(const Tensor& x) {
        std::vector<Tensor> outs;
        for (auto& mb : x.chunk(chunks_, 0)) {
            Tensor h = mb;
            for (auto& s : stages_) h = s(h);
            outs.push_back(h);
        }
        return torch::cat(outs, 0);
    }
    Tensor operator()(const Tensor& x) { return forward(x); }
    size_t num_stages() const { return stages_.size(); }
    int64_t chunks() const { return chunks_; }

 private:
    std::vector<Stage> stages_;
    int64_t chunks_;
};

}  // namespace parallel
}  // namespace nn

namespace distributed {

struct PipelineScheduleConfig {
    int num_stages = 1;
    int num_micros = 1;
    std::string sync_dir;                 // kept for source compatibility; the transport is TCP
    int timeout_ms = 60000;
    int poll_us = 200;
    std::string master_addr = "127.0.0.1";
    int base_port = 29700;
};

namespace detail {
inline void sock_send(int fd, const void* p, size_t n) {
    const char* c = (const char*)p;
    while (n) {
        const ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
        if (k <= 0) throw CollectiveTimeout("pipeline: send failed or timed out");
        c += k;
        n -= (size_t)k;
    }
}
inline void sock_recv(int fd, void* p, size_t n) {
    char* c = (char*)p;
    while (n) {
        const ssize_t k = ::recv(fd, c, n, 0);
        if (k <= 0) throw CollectiveTimeout("pipeline: the neighbouring stage sent nothing within the timeout");
        c += k;
        n -= (size_t)k;
    }
}
inline void sock_options(int fd, int timeout_ms) {
    timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}
// One end of the connection between two neighbouring stages: fp32 tensors with their shape, sends through a queue.
class StageLink {
 public:
    StageLink() = default;
    ~StageLink() { close(); }
    void listen_and_accept(int port, int timeout_ms) {
        const int ls = ::socket(AF_INET, SOCK_STREAM, 0);
        TORCH_CHECK(ls >= 0, "pipeline: socket");
        int one = 1;
        ::setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_addr.s_addr = htonl(INADDR_ANY);
        a.sin_port = htons((uint16_t)port);
        TORCH_CHECK(::bind(ls, (sockaddr*)&a, sizeof(a)) == 0 && ::listen(ls, 1) == 0, "pipeline: cannot listen on port ", port);
        sock_options(ls, timeout_ms);
        fd_ = ::accept(ls, nullptr, nullptr);
        ::close(ls);
        if (fd_ < 0) throw CollectiveTimeout("pipeline: the next stage did not connect within the timeout");
        start(timeout_ms);
    }
    void connect_to(const std::string& addr, int port, int timeout_ms) {
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_port = htons((uint16_t)port);
        TORCH_CHECK(::inet_pton(AF_INET, addr.c_str(), &a.sin_addr) == 1, "pipeline: bad address ", addr);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        for (;;) {
            fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
            TORCH_CHECK(fd_ >= 0, "pipeline: socket");
            if (::connect(fd_, (sockaddr*)&a, sizeof(a)) == 0) break;
            ::close(fd_);
            fd_ = -1;
            if (std::chrono::steady_clock::now() > deadline) throw CollectiveTimeout("pipeline: the previous stage is not listening");
            std::this_thread::sleep_for(std::chrono::milliseconds(10));
        }
        start(timeout_ms);
    }
    void send(const Tensor& t) {
        Tensor h = t.detach().to(torch::kCPU, torch::kFloat).contiguous();
        {
            std::lock_guard<std::mutex> g(m_);
            q_.push_back(std::move(h));
        }
        cv_.notify_one();
    }
    Tensor recv() {
        int64_t nd = 0;
        sock_recv(fd_, &nd, sizeof(nd));
        TORCH_CHECK(nd >= 0 && nd <= 8, "pipeline: bad tensor header");
        std::vector<int64_t> sizes((size_t)nd);
        if (nd) sock_recv(fd_, sizes.data(), sizeof(int64_t) * (size_t)nd);
        Tensor t = torch::empty(sizes, torch::kFloat);
        if (t.numel()) sock_recv(fd_, t.data_ptr(), (size_t)t.numel() * 4);
        return t;
    }
    // Wait until everything queued has gone out (end of a step).
    void flush() {
        std::unique_lock<std::mutex> lk(m_);
        cv_idle_.wait(lk, [&] { return (q_.empty() && !busy_) || failed_; });
        if (failed_) throw CollectiveTimeout("pipeline: a send to the neighbouring stage failed");
    }
    void close() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
        }
        cv_.notify_all();
        if (sender_.joinable()) sender_.join();
        if (fd_ >= 0) ::close(fd_);
        fd_ = -1;
    }
    bool connected() const { return fd_ >= 0; }

 private:
    void start(int timeout_ms) {
        sock_options(fd_, timeout_ms);
        sender_ = std::thread([this] {
            for (;;) {
                Tensor t;
                {
                    std::unique_lock<std::mutex> lk(m_);
                    cv_.wait(lk, [&] { return stop_ || !q_.empty(); });
                    if (q_.empty()) return;
                    t = std::move(q_.front());
                    q_.pop_front();
                    busy_ = true;
                }
                try {
                    const int64_t nd = t.dim();
                    sock_send(fd_, &nd, sizeof(nd));
                    if (nd) sock_send(fd_, t.sizes().data(), sizeof(int64_t) * (size_t)nd);
                    if (t.numel()) sock_send(fd_, t.data_ptr(), (size_t)t.numel() * 4);
                } catch (...) {
                    std::lock_guard<std::mutex> g(m_);
                    failed_ = true;
                }
                {
                    std::lock_guard<std::mutex> g(m_);
                    busy_ = false;
                }
                cv_idle_.notify_all();
            }
        });
    }
    int fd_ = -1;
    std::thread sender_;
    std::deque<Tensor> q_;
    std::mutex m_;
    std::condition_variable cv_, cv_idle_;
    bool stop_ = false, busy_ = false, failed_ = false;
};
}  // namespace detail

template <typename ModuleHolder>
class Pipeline1F1BStage {
 public:
    using LossFn = std::function<Tensor(const Tensor& output, const Tensor& target)>;
    Pipeline1F1BStage(ModuleHolder module, int stage, PipelineScheduleConfig cfg) : module_(std::move(module)), stage_(stage), cfg_(cfg) {
        TORCH_CHECK(stage >= 0 && stage < cfg.num_stages && cfg.num_micros >= 1, "Pipeline1F1BStage: bad stage / schedule");
        // connect to the previous stage first (it is already listening or will be), then accept the next one
        if (!is_first()) prev_.connect_to(cfg_.master_addr, cfg_.base_port + stage_ - 1, cfg_.timeout_ms);
        if (!is_last()) next_.listen_and_accept(cfg_.base_port + stage_, cfg_.timeout_ms);
    }
    bool is_first() const { return stage_ == 0; }
    bool is_last() const { return stage_ == cfg_.num_stages - 1; }
    int stage() const { return stage_; }
    ModuleHolder& module() { return module_; }

    // One training step over num_micros micro-batches.  `inputs`: the micro-batches (first stage only); `targets` and
    // `loss_fn`: last stage only.  Parameter gradients accumulate the mean over the micro-batches.  Returns the mean loss
    // on the last stage and 0 elsewhere.
    double train_step(const std::vector<Tensor>& inputs, const std::vector<Tensor>& targets, const LossFn& loss_fn) {
        const int M = cfg_.num_micros, S = cfg_.num_stages;
        if (is_first()) TORCH_CHECK((int)inputs.size() == M, "Pipeline1F1BStage: the first stage needs ", M, " input micro-batches");
        if (is_last()) TORCH_CHECK((int)targets.size() == M && loss_fn, "Pipeline1F1BStage: the last stage needs targets and a loss");
        xs_.assign(M, Tensor());
        ys_.assign(M, Tensor());
        double loss_sum = 0;
        max_alive_ = 0;
        int alive = 0;
        auto fwd = [&](int i) {
            Tensor x = is_first() ? inputs[i] : prev_.recv().set_requires_grad(true);
            Tensor y = module_->forward(x);
            if (is_last()) {
                y = loss_fn(y, targets[i]) / (double)M;
                loss_sum += y.item<double>();
            } else {
                next_.send(y);
            }
            xs_[i] = x;
            ys_[i] = y;
            max_alive_ = std::max(max_alive_, ++alive);
        };
        auto bwd = [&](int i) {
            if (is_last()) ys_[i].backward();
            else ys_[i].backward(next_.recv().to(ys_[i].device()));
            if (!is_first()) prev_.send(xs_[i].grad());
            xs_[i] = Tensor();
            ys_[i] = Tensor();
            --alive;
        };
        const int warm = std::min(S - stage_ - 1, M);
        for (int i = 0; i < warm; ++i) fwd(i);
        for (int i = 0; i < M - warm; ++i) {
            fwd(warm + i);
            bwd(i);
        }
        for (int i = M - warm; i < M; ++i) bwd(i);
        if (!is_first()) prev_.flush();
        if (!is_last()) next_.flush();
        return loss_sum;
    }
    // The largest number of micro-batches whose activations were alive at once in the last step (S - stage under 1F1B).
    int max_alive_micro_batches() const { return max_alive_; }

 private:
    ModuleHolder module_;
    int stage_;
    PipelineScheduleConfig cfg_;
    detail::StageLink prev_, next_;
    std::vector<Tensor> xs_, ys_;
    int max_alive_ = 0;
};

}  // namespace distributed
}  // namespace promethorch
