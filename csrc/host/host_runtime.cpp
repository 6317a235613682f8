// Host runtime (no CUDA): worker pool, in-process rendezvous all-reduce over float buffers,
// prefetching batch gatherer and durable file replacement.  Plain C ABI for ctypes.
//
// Behaviour follows the reference's host runtime:
//   * worker pool with failure capture        — crates/st-core/src/runtime/golden.rs:237-400
//   * rendezvous all-reduce, uniform failures — crates/spiral-selfsup/src/trainer/distributed.rs:18-430
//   * DataLoader prefetch worker              — crates/st-nn/src/dataset.rs:287-360
//   * atomic_write (tmp + fsync + rename)     — crates/st-core/src/runtime/persistence.rs:21-62
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <fcntl.h>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <unistd.h>
#include <unordered_map>
#include <vector>

#define ST_HOST_API extern "C" __attribute__((visibility("default")))

namespace {
using Clock = std::chrono::steady_clock;

// ------------------------------------------------------------------------------------------------
// worker pool
// ------------------------------------------------------------------------------------------------
typedef int (*TaskFn)(void* arg);   // returns 0 on success; anything else is recorded as a failure

struct Task {
    uint64_t ticket;
    TaskFn fn;
    void* arg;
};

struct Pool {
    std::vector<std::thread> workers;
    std::deque<Task> queue;
    std::mutex mu;
    std::condition_variable cv_work, cv_done;
    std::unordered_map<uint64_t, int> finished;   // ticket → status
    uint64_t next_ticket = 1;
    uint64_t submitted = 0, completed = 0, failed = 0;
    bool stopping = false;

    explicit Pool(int n) {
        for (int i = 0; i < n; ++i) workers.emplace_back([this] { run(); });
    }
    void run() {
        for (;;) {
            Task t;
            {
                std::unique_lock<std::mutex> lk(mu);
                cv_work.wait(lk, [this] { return stopping || !queue.empty(); });
                if (queue.empty()) return;
                t = queue.front();
                queue.pop_front();
            }
            int status = t.fn(t.arg);
            {
                std::lock_guard<std::mutex> lk(mu);
                finished[t.ticket] = status;
                ++completed;
                if (status != 0) ++failed;
            }
            cv_done.notify_all();
        }
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> lk(mu);
            stopping = true;
        }
        cv_work.notify_all();
        for (auto& w : workers) w.join();
    }
};

// ------------------------------------------------------------------------------------------------
// rendezvous
// ------------------------------------------------------------------------------------------------
enum RdvStatus : int {
    RDV_OK = 0,
    RDV_EMPTY_WORLD = 1,
    RDV_RANK_OOB = 2,
    RDV_WORLD_MISMATCH = 3,
    RDV_DUP_RANK = 4,
    RDV_UNKNOWN_RANK = 5,
    RDV_DUP_CONTRIBUTION = 6,
    RDV_LENGTH_MISMATCH = 7,
    RDV_NONFINITE_INPUT = 8,
    RDV_NONFINITE_SUM = 9,
    RDV_PARTICIPANT_LEFT = 10,
    RDV_TIMEOUT = 11,
};

struct Round {
    uint64_t generation = 0;
    std::vector<double> acc;   // double accumulation: the result does not depend on arrival order
                               // to within fp32 rounding of the final value
    std::set<int> contributors;
    int error = RDV_OK;
    int64_t detail[3] = {0, 0, 0};
    bool done = false;
    std::vector<float> result;
};

struct Group {
    std::string id;
    int world = 0;
    std::mutex mu;
    std::condition_variable cv;
    std::set<int> members;
    uint64_t generation = 0;
    std::shared_ptr<Round> round;
};

std::mutex g_reg_mu;
std::map<std::string, std::shared_ptr<Group>> g_registry;

struct Session {
    std::shared_ptr<Group> group;
    int rank;
    bool closed = false;
};

void fail_round(Round& r, int code, int64_t a = 0, int64_t b = 0, int64_t c = 0) {
    r.error = code;
    r.detail[0] = a;
    r.detail[1] = b;
    r.detail[2] = c;
    r.done = true;
}

int collect(Group& g, std::shared_ptr<Round>& rnd, int rank, float* values, int64_t* detail) {
    rnd->contributors.erase(rank);
    if (rnd->contributors.empty() && g.round == rnd) g.round.reset();
    if (rnd->error != RDV_OK) {
        if (detail) std::memcpy(detail, rnd->detail, sizeof(rnd->detail));
        return rnd->error;
    }
    std::memcpy(values, rnd->result.data(), rnd->result.size() * sizeof(float));
    return RDV_OK;
}

// ------------------------------------------------------------------------------------------------
// prefetching batch gatherer
// ------------------------------------------------------------------------------------------------
struct Loader {
    const float* features;
    const float* targets;
    int64_t rows, fcols, tcols;
    std::vector<int64_t> order;
    int64_t batch;
    int depth;
    bool drop_last;
    // ring of produced batches
    struct Slot {
        std::vector<float> x, y;
        int64_t n = 0;
    };
    std::deque<Slot> ready;
    std::mutex mu;
    std::condition_variable cv_space, cv_item;
    std::thread worker;
    bool finished = false, stop = false;

    void produce() {
        int64_t pos = 0;
        const int64_t total = (int64_t)order.size();
        while (pos < total) {
            int64_t n = std::min(batch, total - pos);
            if (n < batch && drop_last) break;
            Slot s;
            s.n = n;
            s.x.resize((size_t)(n * fcols));
            s.y.resize((size_t)(n * tcols));
            for (int64_t i = 0; i < n; ++i) {
                int64_t r = order[(size_t)(pos + i)];
                std::memcpy(&s.x[(size_t)(i * fcols)], features + r * fcols, (size_t)fcols * sizeof(float));
                if (tcols) std::memcpy(&s.y[(size_t)(i * tcols)], targets + r * tcols, (size_t)tcols * sizeof(float));
            }
            pos += n;
            std::unique_lock<std::mutex> lk(mu);
            cv_space.wait(lk, [this] { return stop || (int)ready.size() < depth; });
            if (stop) return;
            ready.emplace_back(std::move(s));
            cv_item.notify_one();
        }
        std::lock_guard<std::mutex> lk(mu);
        finished = true;
        cv_item.notify_all();
    }
    ~Loader() {
        {
            std::lock_guard<std::mutex> lk(mu);
            stop = true;
        }
        cv_space.notify_all();
        if (worker.joinable()) worker.join();
    }
};
}  // namespace

// ================================================================================================
// C ABI
// ================================================================================================
ST_HOST_API void* st_host_pool_create(int workers) {
    if (workers <= 0) workers = (int)std::max(1u, std::thread::hardware_concurrency());
    return new Pool(workers);
}
ST_HOST_API void st_host_pool_destroy(void* p) { delete static_cast<Pool*>(p); }
ST_HOST_API int st_host_pool_workers(void* p) { return (int)static_cast<Pool*>(p)->workers.size(); }

ST_HOST_API uint64_t st_host_pool_submit(void* p, TaskFn fn, void* arg) {
    Pool* pool = static_cast<Pool*>(p);
    uint64_t t;
    {
        std::lock_guard<std::mutex> lk(pool->mu);
        t = pool->next_ticket++;
        pool->queue.push_back(Task{t, fn, arg});
        ++pool->submitted;
    }
    pool->cv_work.notify_one();
    return t;
}

// 0 = finished (status in *status), 1 = still running after timeout_ms, 2 = unknown ticket
ST_HOST_API int st_host_pool_wait(void* p, uint64_t ticket, int64_t timeout_ms, int* status) {
    Pool* pool = static_cast<Pool*>(p);
    std::unique_lock<std::mutex> lk(pool->mu);
    if (ticket == 0 || ticket >= pool->next_ticket) return 2;
    auto pred = [&] { return pool->finished.count(ticket) != 0; };
    if (timeout_ms < 0) {
        pool->cv_done.wait(lk, pred);
    } else if (!pool->cv_done.wait_for(lk, std::chrono::milliseconds(timeout_ms), pred)) {
        return 1;
    }
    if (status) *status = pool->finished[ticket];
    pool->finished.erase(ticket);
    return 0;
}

ST_HOST_API void st_host_pool_stats(void* p, uint64_t* out3) {
    Pool* pool = static_cast<Pool*>(p);
    std::lock_guard<std::mutex> lk(pool->mu);
    out3[0] = pool->submitted;
    out3[1] = pool->completed;
    out3[2] = pool->failed;
}

// ---- rendezvous ---------------------------------------------------------------------------------
ST_HOST_API int st_host_rdv_join(const char* group_id, int rank, int world, void** session, int64_t* detail) {
    if (world <= 0) return RDV_EMPTY_WORLD;
    if (rank < 0 || rank >= world) {
        if (detail) { detail[0] = rank; detail[1] = world; }
        return RDV_RANK_OOB;
    }
    std::shared_ptr<Group> g;
    {
        std::lock_guard<std::mutex> lk(g_reg_mu);
        auto it = g_registry.find(group_id);
        if (it == g_registry.end()) {
            g = std::make_shared<Group>();
            g->id = group_id;
            g->world = world;
            g_registry[group_id] = g;
        } else {
            g = it->second;
        }
    }
    std::lock_guard<std::mutex> lk(g->mu);
    if (g->world != world) {
        if (detail) { detail[0] = g->world; detail[1] = world; }
        return RDV_WORLD_MISMATCH;
    }
    if (g->members.count(rank)) {
        if (detail) detail[0] = rank;
        return RDV_DUP_RANK;
    }
    g->members.insert(rank);
    *session = new Session{g, rank};
    return RDV_OK;
}

ST_HOST_API void st_host_rdv_leave(void* s) {
    Session* ses = static_cast<Session*>(s);
    if (!ses) return;
    if (!ses->closed) {
        ses->closed = true;
        Group& g = *ses->group;
        bool empty;
        {
            std::lock_guard<std::mutex> lk(g.mu);
            g.members.erase(ses->rank);
            if (g.round && !g.round->done) {
                fail_round(*g.round, RDV_PARTICIPANT_LEFT, ses->rank, (int64_t)g.round->generation);
                g.cv.notify_all();
            }
            empty = g.members.empty();
        }
        if (empty) {
            std::lock_guard<std::mutex> lk(g_reg_mu);
            auto it = g_registry.find(g.id);
            if (it != g_registry.end() && it->second.get() == &g) {
                std::lock_guard<std::mutex> lk2(g.mu);
                if (g.members.empty()) g_registry.erase(it);
            }
        }
    }
    delete ses;
}

ST_HOST_API int st_host_rdv_registry_size() {
    std::lock_guard<std::mutex> lk(g_reg_mu);
    return (int)g_registry.size();
}

ST_HOST_API uint64_t st_host_rdv_generation(void* s) {
    Session* ses = static_cast<Session*>(s);
    std::lock_guard<std::mutex> lk(ses->group->mu);
    return ses->group->generation;
}

// Sum `values[0..n)` over all ranks of the group, in place, only if the round completes.
ST_HOST_API int st_host_rdv_all_reduce_sum(void* s, float* values, int64_t n, int64_t timeout_ms, int64_t* detail) {
    Session* ses = static_cast<Session*>(s);
    if (ses->closed) return RDV_UNKNOWN_RANK;
    Group& g = *ses->group;
    const auto started = Clock::now();
    const auto deadline = started + std::chrono::milliseconds(timeout_ms);
    std::unique_lock<std::mutex> lk(g.mu);
    if (!g.members.count(ses->rank)) return RDV_UNKNOWN_RANK;
    std::shared_ptr<Round> rnd = g.round;
    if (!rnd || rnd->done) {
        rnd = std::make_shared<Round>();
        rnd->generation = ++g.generation;
        rnd->acc.assign((size_t)n, 0.0);
        g.round = rnd;
    }
    if (rnd->contributors.count(ses->rank)) {
        if (detail) { detail[0] = ses->rank; detail[1] = (int64_t)rnd->generation; }
        return RDV_DUP_CONTRIBUTION;
    }
    if ((int64_t)rnd->acc.size() != n) {
        fail_round(*rnd, RDV_LENGTH_MISMATCH, (int64_t)rnd->acc.size(), n, ses->rank);
        rnd->contributors.insert(ses->rank);
        g.cv.notify_all();
        return collect(g, rnd, ses->rank, values, detail);
    }
    for (int64_t i = 0; i < n; ++i) {
        if (!std::isfinite(values[i])) {
            fail_round(*rnd, RDV_NONFINITE_INPUT, ses->rank, i);
            rnd->contributors.insert(ses->rank);
            g.cv.notify_all();
            return collect(g, rnd, ses->rank, values, detail);
        }
    }
    for (int64_t i = 0; i < n; ++i) rnd->acc[(size_t)i] += (double)values[i];
    rnd->contributors.insert(ses->rank);
    if ((int)rnd->contributors.size() == g.world) {
        rnd->result.resize((size_t)n);
        int64_t bad = -1;
        for (int64_t i = 0; i < n; ++i) {
            float v = (float)rnd->acc[(size_t)i];
            rnd->result[(size_t)i] = v;
            if (bad < 0 && !std::isfinite(v)) bad = i;
        }
        if (bad >= 0) fail_round(*rnd, RDV_NONFINITE_SUM, bad);
        rnd->done = true;
        g.cv.notify_all();
        return collect(g, rnd, ses->rank, values, detail);
    }
    while (!rnd->done) {
        if (g.cv.wait_until(lk, deadline) == std::cv_status::timeout && !rnd->done) {
            auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(Clock::now() - started).count();
            fail_round(*rnd, RDV_TIMEOUT, (int64_t)rnd->generation, (int64_t)waited);
            g.cv.notify_all();
            break;
        }
    }
    return collect(g, rnd, ses->rank, values, detail);
}

// ---- loader ---------------------------------------------------------------------------------------
ST_HOST_API void* st_host_loader_create(const float* features, const float* targets, int64_t rows, int64_t fcols,
                                        int64_t tcols, const int64_t* order, int64_t order_len, int64_t batch,
                                        int depth, int drop_last) {
    if (batch <= 0 || rows < 0 || fcols <= 0 || depth <= 0) return nullptr;
    for (int64_t i = 0; i < order_len; ++i)
        if (order[i] < 0 || order[i] >= rows) return nullptr;
    Loader* L = new Loader();
    L->features = features;
    L->targets = targets;
    L->rows = rows;
    L->fcols = fcols;
    L->tcols = targets ? tcols : 0;
    L->order.assign(order, order + order_len);
    L->batch = batch;
    L->depth = depth;
    L->drop_last = drop_last != 0;
    L->worker = std::thread([L] { L->produce(); });
    return L;
}

// Copies the next batch into x/y (capacity batch rows); returns its row count, 0 at the end.
ST_HOST_API int64_t st_host_loader_next(void* h, float* x, float* y) {
    Loader* L = static_cast<Loader*>(h);
    Loader::Slot s;
    {
        std::unique_lock<std::mutex> lk(L->mu);
        L->cv_item.wait(lk, [L] { return L->finished || !L->ready.empty(); });
        if (L->ready.empty()) return 0;
        s = std::move(L->ready.front());
        L->ready.pop_front();
    }
    L->cv_space.notify_one();
    std::memcpy(x, s.x.data(), s.x.size() * sizeof(float));
    if (y && !s.y.empty()) std::memcpy(y, s.y.data(), s.y.size() * sizeof(float));
    return s.n;
}
ST_HOST_API void st_host_loader_destroy(void* h) { delete static_cast<Loader*>(h); }

// ---- durable replace ------------------------------------------------------------------------------
// Writes `len` bytes to `<path>.tmp.<pid>`, fsyncs, renames over `path`, fsyncs the directory.
ST_HOST_API int st_host_atomic_write(const char* path, const void* data, int64_t len) {
    std::string target(path);
    std::string tmp = target + ".tmp." + std::to_string((long)getpid());
    int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return 1;
    const char* p = static_cast<const char*>(data);
    int64_t left = len;
    while (left > 0) {
        ssize_t w = ::write(fd, p, (size_t)left);
        if (w <= 0) {
            ::close(fd);
            ::unlink(tmp.c_str());
            return 2;
        }
        p += w;
        left -= w;
    }
    if (::fsync(fd) != 0) {
        ::close(fd);
        ::unlink(tmp.c_str());
        return 3;
    }
    ::close(fd);
    if (::rename(tmp.c_str(), target.c_str()) != 0) {
        ::unlink(tmp.c_str());
        return 4;
    }
    std::string dir = ".";
    auto slash = target.find_last_of('/');
    if (slash != std::string::npos) dir = slash == 0 ? "/" : target.substr(0, slash);
    int dfd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
    if (dfd >= 0) {
        ::fsync(dfd);
        ::close(dfd);
    }
    return 0;
}
