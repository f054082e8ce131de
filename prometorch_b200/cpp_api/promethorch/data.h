// promethorch C++ API: datasets and the data loader.
//
// Dataset / TensorDataset / MapDataset / ConcatDataset / Subset, the samplers, and a DataLoader with
// DataLoaderOptions{batch_size, shuffle, num_workers, prefetch_factor, drop_last, pin_memory, seed} whose worker threads
// fill a bounded queue of collated batches (torch/data/dataloader.h:88-104, 281-470 of the reference).  Batches come out
// in sampler order whatever the number of workers.  DistributedSampler lives in distributed.h.
#pragma once
#include <torch/torch.h>

#include <algorithm>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <random>
#include <thread>
#include <vector>

namespace promethorch {
namespace data {
using Tensor = at::Tensor;

struct Example {
    Tensor data, target;
};
using Batch = Example;

class Dataset {
 public:
    virtual ~Dataset() = default;
    virtual Example get(size_t index) const = 0;
    virtual size_t size() const = 0;
};
using DatasetPtr = std::shared_ptr<const Dataset>;

class TensorDataset : public Dataset {
 public:
    TensorDataset(Tensor data, Tensor target) : data_(std::move(data)), target_(std::move(target)) {
        TORCH_CHECK(data_.size(0) == target_.size(0), "TensorDataset: data and target differ in length");
    }
    Example get(size_t i) const override { return {data_[(int64_t)i], target_[(int64_t)i]}; }
    size_t size() const override { return (size_t)data_.size(0); }

 private:
    Tensor data_, target_;
};
class MapDataset : public Dataset {
 public:
    MapDataset(DatasetPtr base, std::function<Example(Example)> fn) : base_(std::move(base)), fn_(std::move(fn)) {}
    Example get(size_t i) const override { return fn_(base_->get(i)); }
    size_t size() const override { return base_->size(); }

 private:
    DatasetPtr base_;
    std::function<Example(Example)> fn_;
};
class ConcatDataset : public Dataset {
 public:
    explicit ConcatDataset(std::vector<DatasetPtr> parts) : parts_(std::move(parts)) {
        for (auto& p : parts_) total_ += p->size();
    }
    Example get(size_t i) const override {
        for (auto& p : parts_) {
            if (i < p->size()) return p->get(i);
            i -= p->size();
        }
        TORCH_CHECK(false, "ConcatDataset: index out of range");
    }
    size_t size() const override { return total_; }

 private:
    std::vector<DatasetPtr> parts_;
    size_t total_ = 0;
};
class Subset : public Dataset {
 public:
    Subset(DatasetPtr base, std::vector<size_t> indices) : base_(std::move(base)), idx_(std::move(indices)) {}
    Example get(size_t i) const override { return base_->get(idx_.at(i)); }
    size_t size() const override { return idx_.size(); }

 private:
    DatasetPtr base_;
    std::vector<size_t> idx_;
};

// ---- samplers: the order of one epoch
class Sampler {
 public:
    virtual ~Sampler() = default;
    virtual std::vector<size_t> indices() = 0;      // called once per epoch
};
class SequentialSampler : public Sampler {
 public:
    explicit SequentialSampler(size_t n) : n_(n) {}
    std::vector<size_t> indices() override {
        std::vector<size_t> v(n_);
        for (size_t i = 0; i < n_; ++i) v[i] = i;
        return v;
    }

 private:
    size_t n_;
};
class RandomSampler : public Sampler {
 public:
    explicit RandomSampler(size_t n, uint64_t seed = std::random_device{}()) : n_(n), rng_(seed) {}
    std::vector<size_t> indices() override {
        std::vector<size_t> v(n_);
        for (size_t i = 0; i < n_; ++i) v[i] = i;
        std::shuffle(v.begin(), v.end(), rng_);
        return v;
    }

 private:
    size_t n_;
    std::mt19937_64 rng_;
};
class SubsetRandomSampler : public Sampler {
 public:
    SubsetRandomSampler(std::vector<size_t> subset, uint64_t seed = std::random_device{}()) : v_(std::move(subset)), rng_(seed) {}
    std::vector<size_t> indices() override {
        std::shuffle(v_.begin(), v_.end(), rng_);
        return v_;
    }

 private:
    std::vector<size_t> v_;
    std::mt19937_64 rng_;
};
class WeightedRandomSampler : public Sampler {
 public:
    WeightedRandomSampler(std::vector<double> weights, size_t num_samples, uint64_t seed = std::random_device{}())
        : dist_(weights.begin(), weights.end()), n_(num_samples), rng_(seed) {}
    std::vector<size_t> indices() override {
        std::vector<size_t> v(n_);
        for (auto& x : v) x = dist_(rng_);
        return v;
    }

 private:
    std::discrete_distribution<size_t> dist_;
    size_t n_;
    std::mt19937_64 rng_;
};

struct DataLoaderOptions {
    size_t batch_size_v = 1;
    bool shuffle_v = false;
    size_t num_workers_v = 0;
    size_t prefetch_factor_v = 2;
    bool drop_last_v = false;
    bool pin_memory_v = false;
    std::optional<uint64_t> seed_v;
    DataLoaderOptions() = default;
    explicit DataLoaderOptions(size_t batch) : batch_size_v(batch) {}
    DataLoaderOptions& batch_size(size_t v) { batch_size_v = v; return *this; }
    DataLoaderOptions& shuffle(bool v) { shuffle_v = v; return *this; }
    DataLoaderOptions& num_workers(size_t v) { num_workers_v = v; return *this; }
    DataLoaderOptions& prefetch_factor(size_t v) { prefetch_factor_v = v; return *this; }
    DataLoaderOptions& drop_last(bool v) { drop_last_v = v; return *this; }
    DataLoaderOptions& pin_memory(bool v) { pin_memory_v = v; return *this; }
    DataLoaderOptions& seed(uint64_t v) { seed_v = v; return *this; }
};

inline Batch default_collate(const std::vector<Example>& ex) {
    std::vector<Tensor> d, t;
    d.reserve(ex.size());
    t.reserve(ex.size());
    for (auto& e : ex) { d.push_back(e.data); t.push_back(e.target); }
    return {torch::stack(d), torch::stack(t)};
}

// Iterable over the batches of one epoch: `for (auto& batch : loader) ...`; each begin() starts a new epoch.
class DataLoader {
 public:
    using Collate = std::function<Batch(const std::vector<Example>&)>;
    DataLoader(DatasetPtr dataset, DataLoaderOptions opts, std::shared_ptr<Sampler> sampler = nullptr, Collate collate = default_collate)
        : ds_(std::move(dataset)), o_(opts), sampler_(std::move(sampler)), collate_(std::move(collate)) {
        TORCH_CHECK(o_.batch_size_v > 0, "DataLoader: batch_size must be positive");
        if (!sampler_) {
            if (o_.shuffle_v) sampler_ = std::make_shared<RandomSampler>(ds_->size(), o_.seed_v ? *o_.seed_v : std::random_device{}());
            else sampler_ = std::make_shared<SequentialSampler>(ds_->size());
        }
    }
    size_t size() const {        // batches per epoch
        const size_t n = ds_->size(), b = o_.batch_size_v;
        return o_.drop_last_v ? n / b : (n + b - 1) / b;
    }

    class Epoch {
     public:
        Epoch(const DataLoader& dl, std::vector<size_t> order) : dl_(dl), order_(std::move(order)) {
            const size_t b = dl_.o_.batch_size_v, n = order_.size();
            n_batches_ = dl_.o_.drop_last_v ? n / b : (n + b - 1) / b;
            if (dl_.o_.num_workers_v > 0) {
                cap_ = std::max<size_t>(1, dl_.o_.prefetch_factor_v * dl_.o_.num_workers_v);
                for (size_t w = 0; w < dl_.o_.num_workers_v; ++w) workers_.emplace_back([this] { work(); });
            }
        }
        ~Epoch() {
            {
                std::lock_guard<std::mutex> g(m_);
                stop_ = true;
            }
            cv_space_.notify_all();
            cv_ready_.notify_all();
            for (auto& t : workers_) t.join();
        }
        bool has_next() const { return served_ < n_batches_; }
        Batch next() {
            TORCH_CHECK(has_next(), "DataLoader: epoch exhausted");
            if (workers_.empty()) return make(served_++);
            std::unique_lock<std::mutex> lk(m_);
            const size_t want = served_++;
            cv_space_.notify_all();
            cv_ready_.wait(lk, [&] { return ready_.count(want) > 0; });
            Batch b = std::move(ready_[want]);
            ready_.erase(want);
            lk.unlock();
            cv_space_.notify_all();
            return b;
        }

     private:
        Batch make(size_t bi) const {
            const size_t b = dl_.o_.batch_size_v, lo = bi * b, hi = std::min(order_.size(), lo + b);
            std::vector<Example> ex;
            ex.reserve(hi - lo);
            for (size_t i = lo; i < hi; ++i) ex.push_back(dl_.ds_->get(order_[i]));
            Batch out = dl_.collate_(ex);
            if (dl_.o_.pin_memory_v && torch::cuda::is_available()) { out.data = out.data.pin_memory(); out.target = out.target.pin_memory(); }
            return out;
        }
        void work() {
            for (;;) {
                size_t bi;
                {
                    std::unique_lock<std::mutex> lk(m_);
                    // bounded look-ahead: at most `cap_` batches beyond the one the consumer waits for
                    cv_space_.wait(lk, [&] { return stop_ || next_ >= n_batches_ || next_ < served_ + cap_; });
                    if (stop_ || next_ >= n_batches_) return;
                    bi = next_++;
                }
                Batch b = make(bi);
                {
                    std::lock_guard<std::mutex> g(m_);
                    ready_[bi] = std::move(b);
                }
                cv_ready_.notify_all();
            }
        }
        const DataLoader& dl_;
        std::vector<size_t> order_;
        size_t n_batches_ = 0, served_ = 0, next_ = 0, cap_ = 1;
        std::vector<std::thread> workers_;
        std::map<size_t, Batch> ready_;
        std::mutex m_;
        std::condition_variable cv_ready_, cv_space_;
        bool stop_ = false;
    };

    // range-for support
    class iterator {
     public:
        iterator() = default;
        explicit iterator(std::shared_ptr<Epoch> e) : e_(std::move(e)) { advance(); }
        Batch& operator*() { return cur_; }
        Batch* operator->() { return &cur_; }
        iterator& operator++() { advance(); return *this; }
        bool operator!=(const iterator& o) const { return done_ != o.done_; }

     private:
        void advance() {
            if (e_ && e_->has_next()) cur_ = e_->next();
            else done_ = true;
        }
        std::shared_ptr<Epoch> e_;
        Batch cur_;
        bool done_ = false;
    };
    iterator begin() { return iterator(std::make_shared<Epoch>(*this, sampler_->indices())); }
    iterator end() {
        iterator it;
        ++it;
        return it;
    }

 private:
    friend class Epoch;
    DatasetPtr ds_;
    DataLoaderOptions o_;
    std::shared_ptr<Sampler> sampler_;
    Collate collate_;
};

}  // namespace data
}  // namespace promethorch
