// Implementation of the MPI subset declared in mpi.h (see there).  One process = one rank; every pair of ranks shares
// one Unix-domain stream socket in the abstract namespace ("\0mpishim-<job>-<rank>"), so no file is created anywhere.
#include "mpi.h"

#include <errno.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Msg { int src, tag; std::vector<char> data; };
struct Pending { void* buf; long cap; int src, tag; bool active; };

// All state lives in one object on the heap that is never destroyed: the receiver thread may still be running when a
// process leaves through exit() without MPI_Finalize (the reference does that on errors), and must not find its mutexes
// or its mailbox destructed under it.
struct State {
    int rank = 0, size = 1;
    std::string job;
    std::vector<int> fd;
    std::vector<std::unique_ptr<std::mutex>> send_mu;
    std::mutex mu;                      // mailbox and request table
    std::condition_variable cv;
    std::list<Msg> box;
    std::vector<Pending> req;
    std::thread* receiver = nullptr;
    std::atomic<bool> stop{false};
    bool inited = false;
};
State& S = *new State;
#define g_rank S.rank
#define g_size S.size
#define g_job S.job
#define g_fd S.fd
#define g_send_mu S.send_mu
#define g_mu S.mu
#define g_cv S.cv
#define g_box S.box
#define g_req S.req
#define g_receiver S.receiver
#define g_stop S.stop
#define g_inited S.inited

enum { TAG_BARRIER_IN = -2, TAG_BARRIER_OUT = -3, TAG_BCAST = -4, TAG_REDUCE = -5, TAG_GATHER = -6 };

[[noreturn]] void die(const char* what) {
    fprintf(stderr, "mpi_shim (rank %d of %d): %s: %s\n", g_rank, g_size, what, strerror(errno));
    _exit(70);
}

int type_size(MPI_Datatype t) {
    switch (t) {
        case MPI_CHAR: case MPI_UNSIGNED_CHAR: case MPI_INT8_T: case MPI_BYTE: return 1;
        case MPI_UINT16_T: return 2;
        case MPI_INT: case MPI_UNSIGNED: case MPI_FLOAT: case MPI_INT32_T: case MPI_UINT32_T: return 4;
        case MPI_LONG: case MPI_UNSIGNED_LONG: case MPI_DOUBLE: case MPI_UINT64_T: case MPI_INT64_T: return 8;
        default: fprintf(stderr, "mpi_shim: unsupported datatype %d\n", t); _exit(71);
    }
}

void write_all(int fd, const void* p, size_t n) {
    const char* c = (const char*)p;
    while (n) {
        ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
        if (k < 0) { if (errno == EINTR) continue; die("send"); }
        c += k; n -= (size_t)k;
    }
}

bool read_all(int fd, void* p, size_t n) {      // false: peer closed before the first byte
    char* c = (char*)p;
    size_t got = 0;
    while (got < n) {
        ssize_t k = ::recv(fd, c + got, n - got, 0);
        if (k == 0) { if (got == 0) return false; errno = ECONNRESET; die("peer closed in the middle of a message"); }
        if (k < 0) { if (errno == EINTR) continue; die("recv"); }
        got += (size_t)k;
    }
    return true;
}

sockaddr_un address_of(int rank, socklen_t* len) {
    sockaddr_un a;
    memset(&a, 0, sizeof a);
    a.sun_family = AF_UNIX;
    const std::string name = "mpishim-" + g_job + "-" + std::to_string(rank);
    memcpy(a.sun_path + 1, name.data(), name.size());          // leading NUL: abstract namespace
    *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
    return a;
}

void deliver(Msg&& m) {
    { std::lock_guard<std::mutex> l(g_mu); g_box.push_back(std::move(m)); }
    g_cv.notify_all();
}

void receiver_loop() {
    std::vector<pollfd> pf;
    for (int r = 0; r < g_size; ++r) if (r != g_rank) pf.push_back({g_fd[r], POLLIN, 0});
    size_t open_peers = pf.size();
    while (!g_stop.load() && open_peers) {
        const int n = poll(pf.data(), pf.size(), 200);
        if (n < 0) { if (errno == EINTR) continue; die("poll"); }
        for (auto& p : pf) {
            if (p.fd < 0 || !(p.revents & (POLLIN | POLLHUP))) continue;
            int32_t head[2];
            uint64_t nbytes;
            if (!read_all(p.fd, head, sizeof head)) { p.fd = -1; --open_peers; continue; }   // peer finalised
            read_all(p.fd, &nbytes, sizeof nbytes);
            Msg m{head[0], head[1], std::vector<char>((size_t)nbytes)};
            if (nbytes) read_all(p.fd, m.data.data(), (size_t)nbytes);
            deliver(std::move(m));
        }
    }
}

void send_bytes(const void* buf, size_t n, int dest, int tag) {
    if (dest < 0 || dest >= g_size) { errno = EINVAL; die("send to a rank outside the world"); }
    if (dest == g_rank) { deliver(Msg{g_rank, tag, std::vector<char>((const char*)buf, (const char*)buf + n)}); return; }
    std::lock_guard<std::mutex> l(*g_send_mu[dest]);
    const int32_t head[2] = {g_rank, tag};
    const uint64_t nbytes = n;
    write_all(g_fd[dest], head, sizeof head);
    write_all(g_fd[dest], &nbytes, sizeof nbytes);
    if (n) write_all(g_fd[dest], buf, n);
}

bool matches(const Msg& m, int src, int tag) {
    if (src != MPI_ANY_SOURCE && m.src != src) return false;
    if (tag == MPI_ANY_TAG) return m.tag >= 0;               // internal (negative) tags never match a wildcard
    return m.tag == tag;
}

// caller holds g_mu
bool try_take(void* buf, long cap, int src, int tag, MPI_Status* st) {
    for (auto it = g_box.begin(); it != g_box.end(); ++it) {
        if (!matches(*it, src, tag)) continue;
        if ((long)it->data.size() > cap) { fprintf(stderr, "mpi_shim (rank %d): message of %zu bytes from %d (tag %d) does not fit %ld\n", g_rank, it->data.size(), it->src, it->tag, cap); _exit(72); }
        if (!it->data.empty()) memcpy(buf, it->data.data(), it->data.size());
        if (st) { st->MPI_SOURCE = it->src; st->MPI_TAG = it->tag; st->MPI_ERROR = MPI_SUCCESS; st->count_bytes_ = (long)it->data.size(); }
        g_box.erase(it);
        return true;
    }
    return false;
}

void recv_bytes(void* buf, long cap, int src, int tag, MPI_Status* st) {
    std::unique_lock<std::mutex> l(g_mu);
    while (!try_take(buf, cap, src, tag, st)) g_cv.wait(l);
}

void connect_world() {
    g_fd.assign(g_size, -1);
    for (int r = 0; r < g_size; ++r) g_send_mu.emplace_back(new std::mutex);
    if (g_size == 1) return;
    const int lst = socket(AF_UNIX, SOCK_STREAM, 0);
    if (lst < 0) die("socket");
    socklen_t len;
    sockaddr_un me = address_of(g_rank, &len);
    if (bind(lst, (sockaddr*)&me, len) < 0) die("bind");
    if (listen(lst, g_size) < 0) die("listen");
    for (int p = 0; p < g_rank; ++p) {               // connect to every lower rank (it may not listen yet: retry)
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(120);
        for (;;) {
            const int fd = socket(AF_UNIX, SOCK_STREAM, 0);
            if (fd < 0) die("socket");
            sockaddr_un a = address_of(p, &len);
            if (connect(fd, (sockaddr*)&a, len) == 0) {
                const int32_t id = g_rank;
                write_all(fd, &id, sizeof id);
                g_fd[p] = fd;
                break;
            }
            close(fd);
            if (std::chrono::steady_clock::now() > deadline) die("connect (peer never appeared)");
            std::this_thread::sleep_for(std::chrono::milliseconds(20));
        }
    }
    for (int k = g_rank + 1; k < g_size; ++k) {       // accept every higher rank
        const int fd = accept(lst, nullptr, nullptr);
        if (fd < 0) die("accept");
        int32_t id = -1;
        if (!read_all(fd, &id, sizeof id) || id <= g_rank || id >= g_size || g_fd[id] != -1) { errno = EPROTO; die("handshake"); }
        g_fd[id] = fd;
    }
    close(lst);
    g_receiver = new std::thread(receiver_loop);
}

template <class T>
void reduce_into(T* acc, const T* x, int n, MPI_Op op) {
    for (int i = 0; i < n; ++i) acc[i] = op == MPI_SUM ? acc[i] + x[i] : op == MPI_MAX ? (x[i] > acc[i] ? x[i] : acc[i]) : (x[i] < acc[i] ? x[i] : acc[i]);
}

void reduce_typed(void* acc, const void* x, int n, MPI_Datatype t, MPI_Op op) {
    switch (t) {
        case MPI_DOUBLE: reduce_into((double*)acc, (const double*)x, n, op); break;
        case MPI_FLOAT: reduce_into((float*)acc, (const float*)x, n, op); break;
        case MPI_INT: case MPI_INT32_T: reduce_into((int32_t*)acc, (const int32_t*)x, n, op); break;
        case MPI_UNSIGNED: case MPI_UINT32_T: reduce_into((uint32_t*)acc, (const uint32_t*)x, n, op); break;
        case MPI_LONG: case MPI_INT64_T: reduce_into((int64_t*)acc, (const int64_t*)x, n, op); break;
        case MPI_UNSIGNED_LONG: case MPI_UINT64_T: reduce_into((uint64_t*)acc, (const uint64_t*)x, n, op); break;
        default: fprintf(stderr, "mpi_shim: reduction on datatype %d is not supported\n", t); _exit(73);
    }
}

}  // namespace

int MPI_Init_thread(int*, char***, int required, int* provided) {
    if (provided) *provided = required;
    if (g_inited) return MPI_SUCCESS;
    g_inited = true;
    const char* r = getenv("MPISHIM_RANK");
    const char* s = getenv("MPISHIM_SIZE");
    const char* j = getenv("MPISHIM_JOB");
    if (r && s && j) { g_rank = atoi(r); g_size = atoi(s); g_job = j; }
    if (g_size < 1 || g_rank < 0 || g_rank >= g_size) { errno = EINVAL; die("bad MPISHIM_RANK / MPISHIM_SIZE"); }
    connect_world();
    return MPI_SUCCESS;
}
int MPI_Init(int* argc, char*** argv) { return MPI_Init_thread(argc, argv, MPI_THREAD_SINGLE, nullptr); }

int MPI_Finalize() {
    if (!g_inited) return MPI_SUCCESS;
    MPI_Barrier(MPI_COMM_WORLD);
    g_stop.store(true);
    for (int r = 0; r < g_size; ++r) if (g_fd[r] >= 0) shutdown(g_fd[r], SHUT_WR);
    if (g_receiver) { g_receiver->join(); delete g_receiver; g_receiver = nullptr; }
    for (int r = 0; r < g_size; ++r) if (g_fd[r] >= 0) { close(g_fd[r]); g_fd[r] = -1; }
    return MPI_SUCCESS;
}
int MPI_Abort(MPI_Comm, int code) { _exit(code ? code : 1); }
int MPI_Comm_rank(MPI_Comm, int* rank) { *rank = g_rank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm, int* size) { *size = g_size; return MPI_SUCCESS; }
int MPI_Get_processor_name(char* name, int* len) { strcpy(name, "localhost"); *len = 9; return MPI_SUCCESS; }

int MPI_Send(const void* buf, int count, MPI_Datatype type, int dest, int tag, MPI_Comm) {
    send_bytes(buf, (size_t)count * type_size(type), dest, tag);
    return MPI_SUCCESS;
}
int MPI_Recv(void* buf, int count, MPI_Datatype type, int source, int tag, MPI_Comm, MPI_Status* status) {
    recv_bytes(buf, (long)count * type_size(type), source, tag, status);
    return MPI_SUCCESS;
}
int MPI_Isend(const void* buf, int count, MPI_Datatype type, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
    MPI_Send(buf, count, type, dest, tag, comm);          // eager: the data is on its way when this returns
    *req = MPI_REQUEST_NULL;
    return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype type, int source, int tag, MPI_Comm, MPI_Request* req) {
    std::lock_guard<std::mutex> l(g_mu);
    size_t slot = 0;
    while (slot < g_req.size() && g_req[slot].active) ++slot;
    if (slot == g_req.size()) g_req.push_back(Pending{});
    g_req[slot] = Pending{buf, (long)count * type_size(type), source, tag, true};
    *req = (MPI_Request)slot;
    return MPI_SUCCESS;
}
int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status) {
    if (*req == MPI_REQUEST_NULL) { *flag = 1; return MPI_SUCCESS; }
    std::lock_guard<std::mutex> l(g_mu);
    Pending& p = g_req[(size_t)*req];
    *flag = try_take(p.buf, p.cap, p.src, p.tag, status) ? 1 : 0;
    if (*flag) { p.active = false; *req = MPI_REQUEST_NULL; }
    return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* req, MPI_Status* status) {
    if (*req == MPI_REQUEST_NULL) return MPI_SUCCESS;
    std::unique_lock<std::mutex> l(g_mu);
    Pending& p = g_req[(size_t)*req];
    while (!try_take(p.buf, p.cap, p.src, p.tag, status)) g_cv.wait(l);
    p.active = false;
    *req = MPI_REQUEST_NULL;
    return MPI_SUCCESS;
}
int MPI_Cancel(MPI_Request* req) {
    if (*req == MPI_REQUEST_NULL) return MPI_SUCCESS;
    std::lock_guard<std::mutex> l(g_mu);
    g_req[(size_t)*req].active = false;
    *req = MPI_REQUEST_NULL;
    return MPI_SUCCESS;
}
int MPI_Request_free(MPI_Request* req) { return MPI_Cancel(req); }
int MPI_Get_count(const MPI_Status* status, MPI_Datatype type, int* count) {
    *count = (int)(status->count_bytes_ / type_size(type));
    return MPI_SUCCESS;
}

int MPI_Barrier(MPI_Comm) {
    if (g_size == 1) return MPI_SUCCESS;
    char c = 0;
    if (g_rank == 0) {
        for (int r = 1; r < g_size; ++r) recv_bytes(&c, 1, r, TAG_BARRIER_IN, nullptr);
        for (int r = 1; r < g_size; ++r) send_bytes(&c, 1, r, TAG_BARRIER_OUT);
    } else {
        send_bytes(&c, 1, 0, TAG_BARRIER_IN);
        recv_bytes(&c, 1, 0, TAG_BARRIER_OUT, nullptr);
    }
    return MPI_SUCCESS;
}
int MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm) {
    if (g_size == 1) return MPI_SUCCESS;
    const size_t n = (size_t)count * type_size(type);
    if (g_rank == root) { for (int r = 0; r < g_size; ++r) if (r != root) send_bytes(buf, n, r, TAG_BCAST); }
    else recv_bytes(buf, (long)n, root, TAG_BCAST, nullptr);
    return MPI_SUCCESS;
}
int MPI_Allreduce(const void* in, void* out, int count, MPI_Datatype type, MPI_Op op, MPI_Comm comm) {
    const size_t n = (size_t)count * type_size(type);
    if (in != MPI_IN_PLACE && in != out) memcpy(out, in, n);
    if (g_size == 1) return MPI_SUCCESS;
    if (g_rank == 0) {
        std::vector<char> tmp(n);
        for (int r = 1; r < g_size; ++r) {               // rank order: the result does not depend on arrival order
            recv_bytes(tmp.data(), (long)n, r, TAG_REDUCE, nullptr);
            reduce_typed(out, tmp.data(), count, type, op);
        }
    } else send_bytes(out, n, 0, TAG_REDUCE);
    return MPI_Bcast(out, count, type, 0, comm);
}
int MPI_Allgather(const void* in, int count, MPI_Datatype type, void* out, int, MPI_Datatype, MPI_Comm comm) {
    const size_t n = (size_t)count * type_size(type);
    char* o = (char*)out;
    if (in != MPI_IN_PLACE) memcpy(o + n * g_rank, in, n);
    if (g_size == 1) return MPI_SUCCESS;
    if (g_rank == 0) { for (int r = 1; r < g_size; ++r) recv_bytes(o + n * r, (long)n, r, TAG_GATHER, nullptr); }
    else send_bytes(o + n * g_rank, n, 0, TAG_GATHER);
    return MPI_Bcast(out, count * g_size, type, 0, comm);
}

int MPI_Get_address(const void* location, MPI_Aint* address) { *address = (MPI_Aint)location; return MPI_SUCCESS; }
int MPI_Type_create_struct(int, const int*, const MPI_Aint*, const MPI_Datatype*, MPI_Datatype* newtype) { *newtype = MPI_BYTE; return MPI_SUCCESS; }
int MPI_Type_commit(MPI_Datatype*) { return MPI_SUCCESS; }
