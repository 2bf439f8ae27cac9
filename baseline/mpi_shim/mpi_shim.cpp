// Implementation of the single-node MPI subset declared in mpi.h.
//
// Transport: one single-producer/single-consumer byte ring per ordered rank
// pair in a POSIX shared-memory segment.  A message is a 24-byte header
// {context, tag, bytes} followed by its payload, streamed through the ring, so
// messages may be larger than the ring.  Every blocking call drains the
// caller's incoming rings while it waits (into posted receives, or into an
// unexpected-message queue), so cyclic blocking sends cannot deadlock.
// Collectives are written on top of point-to-point with reserved tags.
#include "mpi.h"

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <fcntl.h>
#include <map>
#include <memory>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

constexpr size_t RING_CAP = 1u << 21;  // 2 MiB per ordered pair
constexpr uint32_t MAGIC = 0x53503344;
constexpr int TAG_COLL = -1000;         // internal collectives use tags below this

struct alignas(64) Ring {
    std::atomic<uint64_t> head;  // bytes produced
    char pad0[56];
    std::atomic<uint64_t> tail;  // bytes consumed
    char pad1[56];
    char data[RING_CAP];
};

struct ShmHeader {
    std::atomic<uint32_t> magic;
    uint32_t nranks;
    std::atomic<uint32_t> attached;
    std::atomic<uint32_t> finalized;
    char pad[48];
};

struct MsgHeader { uint64_t ctx; int64_t tag; uint64_t bytes; };

struct Unexpected {
    uint64_t ctx; int64_t tag; int src_world;
    std::vector<char> data;
    bool complete = false;
    struct Req* attached = nullptr;
};

struct Req {
    void* buf; size_t cap; uint64_t ctx; int64_t tag; int src_world;
    bool done = false, matched = false;
    size_t got = 0;
};

struct InState {
    int phase = 0;  // 0 header, 1 payload
    MsgHeader hdr{};
    size_t got = 0;
    char hbuf[sizeof(MsgHeader)];
    Req* req = nullptr;
    std::shared_ptr<Unexpected> unex;
};

struct Comm {
    uint64_t ctx = 0;
    std::vector<int> world;  // comm rank -> world rank
    int myrank = -1;
    int ndims = 0;
    std::vector<int> dims, coords;
    uint64_t children = 0;
    std::vector<int> nb_in, nb_out;  // dist graph neighbours (comm ranks)
};

struct DType {
    size_t size = 0;                        // bytes of one element when packed
    std::vector<std::pair<ptrdiff_t, size_t>> blocks;  // (byte offset, byte length); empty = contiguous
};

int g_rank = -1, g_size = 0;
ShmHeader* g_hdr = nullptr;
Ring* g_rings = nullptr;
std::string g_shm_name;
size_t g_shm_bytes = 0;
std::vector<InState> g_in;
std::deque<Req*> g_posted;
std::deque<std::shared_ptr<Unexpected>> g_unexpected;
std::map<int, Comm> g_comms;
std::map<int, DType> g_types;
std::map<int, Req*> g_reqs;
std::map<int, FILE*> g_files;
int g_next_comm = 2, g_next_type = 100, g_next_req = 1, g_next_file = 1;

Ring& ring(int src, int dst) { return g_rings[(size_t)src * g_size + dst]; }

[[noreturn]] void die(const char* msg) {
    fprintf(stderr, "[mpi shim rank %d] %s\n", g_rank, msg);
    _exit(3);
}

uint64_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31);
}

size_t type_size(MPI_Datatype t) {
    switch (t) {
        case MPI_CHAR: case MPI_BYTE: return 1;
        case MPI_INT: case MPI_UNSIGNED: case MPI_FLOAT: return 4;
        case MPI_UNSIGNED_LONG: case MPI_DOUBLE: case MPI_2INT: case MPI_LONG_LONG: return 8;
        default: {
            auto it = g_types.find(t);
            if (it == g_types.end()) die("unknown datatype");
            return it->second.size;
        }
    }
}

// ---- progress engine ---------------------------------------------------------
void deliver_complete(InState& st) {
    if (st.req) { st.req->done = true; st.req = nullptr; }
    else if (st.unex) {
        st.unex->complete = true;
        if (st.unex->attached) {
            Req* r = st.unex->attached;
            if (st.unex->data.size() > r->cap) die("message longer than receive buffer");
            memcpy(r->buf, st.unex->data.data(), st.unex->data.size());
            r->done = true;
            g_unexpected.erase(std::find(g_unexpected.begin(), g_unexpected.end(), st.unex));
        }
        st.unex.reset();
    }
    st.phase = 0; st.got = 0;
}

bool progress_from(int src) {
    Ring& r = ring(src, g_rank);
    InState& st = g_in[src];
    bool any = false;
    for (;;) {
        const uint64_t head = r.head.load(std::memory_order_acquire);
        uint64_t tail = r.tail.load(std::memory_order_relaxed);
        size_t avail = (size_t)(head - tail);
        if (!avail) break;
        any = true;
        char* dst; size_t want;
        if (st.phase == 0) { dst = st.hbuf + st.got; want = sizeof(MsgHeader) - st.got; }
        else {
            char* base = st.req ? (char*)st.req->buf : st.unex->data.data();
            dst = base + st.got; want = (size_t)st.hdr.bytes - st.got;
        }
        size_t n = std::min(avail, want);
        size_t pos = (size_t)(tail % RING_CAP);
        size_t first = std::min(n, RING_CAP - pos);
        memcpy(dst, r.data + pos, first);
        if (n > first) memcpy(dst + first, r.data, n - first);
        r.tail.store(tail + n, std::memory_order_release);
        st.got += n;
        if (st.phase == 0 && st.got == sizeof(MsgHeader)) {
            memcpy(&st.hdr, st.hbuf, sizeof(MsgHeader));
            st.phase = 1; st.got = 0; st.req = nullptr; st.unex.reset();
            for (auto it = g_posted.begin(); it != g_posted.end(); ++it) {
                Req* q = *it;
                if (!q->matched && q->ctx == st.hdr.ctx && q->src_world == src && q->tag == st.hdr.tag) {
                    if (st.hdr.bytes > q->cap) die("message longer than receive buffer");
                    q->matched = true; st.req = q; g_posted.erase(it); break;
                }
            }
            if (!st.req) {
                st.unex = std::make_shared<Unexpected>();
                st.unex->ctx = st.hdr.ctx; st.unex->tag = st.hdr.tag; st.unex->src_world = src;
                st.unex->data.resize((size_t)st.hdr.bytes);
                g_unexpected.push_back(st.unex);
            }
            if (st.hdr.bytes == 0) deliver_complete(st);
        } else if (st.phase == 1 && st.got == (size_t)st.hdr.bytes) {
            deliver_complete(st);
        }
    }
    return any;
}

void progress() {
    for (int s = 0; s < g_size; ++s) progress_from(s);
}

void idle(unsigned& spins) {
    if (++spins > 200) { sched_yield(); }
    else { __builtin_ia32_pause(); }
}

void ring_write(int dst, const void* p, size_t n) {
    Ring& r = ring(g_rank, dst);
    const char* src = (const char*)p;
    unsigned spins = 0;
    while (n) {
        uint64_t head = r.head.load(std::memory_order_relaxed);
        uint64_t tail = r.tail.load(std::memory_order_acquire);
        size_t space = RING_CAP - (size_t)(head - tail);
        if (!space) { progress(); idle(spins); continue; }
        spins = 0;
        size_t m = std::min(space, n);
        size_t pos = (size_t)(head % RING_CAP);
        size_t first = std::min(m, RING_CAP - pos);
        memcpy(r.data + pos, src, first);
        if (m > first) memcpy(r.data, src + first, m - first);
        r.head.store(head + m, std::memory_order_release);
        src += m; n -= m;
    }
}

void raw_send(int dst_world, uint64_t ctx, int64_t tag, const void* buf, size_t bytes) {
    MsgHeader h{ctx, tag, bytes};
    ring_write(dst_world, &h, sizeof h);
    ring_write(dst_world, buf, bytes);
}

Req* raw_irecv(int src_world, uint64_t ctx, int64_t tag, void* buf, size_t cap) {
    Req* q = new Req{buf, cap, ctx, tag, src_world};
    progress();
    for (auto it = g_unexpected.begin(); it != g_unexpected.end(); ++it) {
        auto& u = *it;
        if (u->attached == nullptr && u->ctx == ctx && u->src_world == src_world && u->tag == tag) {
            q->matched = true;
            if (u->complete) {
                if (u->data.size() > cap) die("message longer than receive buffer");
                memcpy(buf, u->data.data(), u->data.size());
                q->done = true;
                g_unexpected.erase(it);
            } else u->attached = q;
            return q;
        }
    }
    g_posted.push_back(q);
    return q;
}

void raw_wait(Req* q) {
    unsigned spins = 0;
    while (!q->done) { progress(); if (!q->done) idle(spins); }
    delete q;
}

void raw_recv(int src_world, uint64_t ctx, int64_t tag, void* buf, size_t cap) { raw_wait(raw_irecv(src_world, ctx, tag, buf, cap)); }

Comm& comm_of(MPI_Comm c) {
    auto it = g_comms.find(c);
    if (it == g_comms.end()) die("invalid communicator");
    return it->second;
}

// packs `count` elements of type t starting at buf into a contiguous vector (only when derived)
const void* pack(const void* buf, int count, MPI_Datatype t, std::vector<char>& tmp, size_t* bytes) {
    auto it = g_types.find(t);
    if (it == g_types.end() || it->second.blocks.empty()) { *bytes = (size_t)count * type_size(t); return buf; }
    const DType& d = it->second;
    tmp.resize((size_t)count * d.size);
    char* out = tmp.data();
    for (int c = 0; c < count; ++c)  // count > 1 of an indexed type is not used by the callers; extent = packed size
        for (auto& b : d.blocks) { memcpy(out, (const char*)buf + b.first, b.second); out += b.second; }
    *bytes = tmp.size();
    return tmp.data();
}

template <typename T> void reduce_typed(T* acc, const T* in, size_t n, MPI_Op op) {
    for (size_t i = 0; i < n; ++i) {
        if (op == MPI_SUM) acc[i] += in[i];
        else if (op == MPI_MAX) acc[i] = std::max(acc[i], in[i]);
        else if (op == MPI_MIN) acc[i] = std::min(acc[i], in[i]);
    }
}

void reduce_into(void* acc, const void* in, int count, MPI_Datatype t, MPI_Op op) {
    if (op == MPI_MAXLOC && t == MPI_2INT) {
        int* a = (int*)acc; const int* b = (const int*)in;
        for (int i = 0; i < count; ++i)
            if (b[2 * i] > a[2 * i] || (b[2 * i] == a[2 * i] && b[2 * i + 1] < a[2 * i + 1])) { a[2 * i] = b[2 * i]; a[2 * i + 1] = b[2 * i + 1]; }
        return;
    }
    switch (t) {
        case MPI_INT: reduce_typed((int*)acc, (const int*)in, count, op); break;
        case MPI_UNSIGNED: reduce_typed((unsigned*)acc, (const unsigned*)in, count, op); break;
        case MPI_UNSIGNED_LONG: reduce_typed((unsigned long*)acc, (const unsigned long*)in, count, op); break;
        case MPI_LONG_LONG: reduce_typed((long long*)acc, (const long long*)in, count, op); break;
        case MPI_DOUBLE: reduce_typed((double*)acc, (const double*)in, count, op); break;
        case MPI_FLOAT: reduce_typed((float*)acc, (const float*)in, count, op); break;
        default: die("unsupported reduction datatype");
    }
}

int new_comm(Comm&& c) { int id = g_next_comm++; g_comms[id] = std::move(c); return id; }

}  // namespace

extern "C" {

int MPI_Init(int*, char***) {
    const char* r = getenv("SP3MPI_RANK"); const char* s = getenv("SP3MPI_SIZE"); const char* j = getenv("SP3MPI_JOB");
    g_rank = r ? atoi(r) : 0; g_size = s ? atoi(s) : 1;
    g_shm_name = std::string("/sp3mpi_") + (j ? j : std::to_string(getpid()));
    g_shm_bytes = sizeof(ShmHeader) + sizeof(Ring) * (size_t)g_size * g_size;
    int fd = -1;
    if (g_rank == 0) {
        shm_unlink(g_shm_name.c_str());
        fd = shm_open(g_shm_name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0 || ftruncate(fd, (off_t)g_shm_bytes) != 0) die("cannot create shared memory segment");
    } else {
        for (int tries = 0; tries < 60000; ++tries) {
            fd = shm_open(g_shm_name.c_str(), O_RDWR, 0600);
            if (fd >= 0) { struct stat st; if (fstat(fd, &st) == 0 && (size_t)st.st_size >= g_shm_bytes) break; close(fd); fd = -1; }
            usleep(1000);
        }
        if (fd < 0) die("shared memory segment did not appear");
    }
    void* p = mmap(nullptr, g_shm_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) die("mmap failed");
    g_hdr = (ShmHeader*)p;
    g_rings = (Ring*)((char*)p + sizeof(ShmHeader));
    if (g_rank == 0) {  // a fresh segment is zero filled: ring heads/tails start at 0
        g_hdr->nranks = g_size; g_hdr->attached.store(0); g_hdr->finalized.store(0);
        g_hdr->magic.store(MAGIC, std::memory_order_release);
    } else {
        while (g_hdr->magic.load(std::memory_order_acquire) != MAGIC) usleep(100);
    }
    g_hdr->attached.fetch_add(1);
    while (g_hdr->attached.load() < (uint32_t)g_size) usleep(100);
    g_in.assign(g_size, InState{});
    Comm w; w.ctx = 1; w.myrank = g_rank;
    for (int i = 0; i < g_size; ++i) w.world.push_back(i);
    g_comms[MPI_COMM_WORLD] = std::move(w);
    return MPI_SUCCESS;
}

int MPI_Finalize(void) {
    MPI_Barrier(MPI_COMM_WORLD);
    g_hdr->finalized.fetch_add(1);
    if (g_rank == 0) {
        while (g_hdr->finalized.load() < (uint32_t)g_size) usleep(100);
        shm_unlink(g_shm_name.c_str());
    }
    munmap((void*)g_hdr, g_shm_bytes);
    return MPI_SUCCESS;
}

int MPI_Abort(MPI_Comm, int code) { _exit(code ? code : 1); }
double MPI_Wtime(void) { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
int MPI_Comm_rank(MPI_Comm c, int* r) { *r = comm_of(c).myrank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm c, int* s) { *s = (int)comm_of(c).world.size(); return MPI_SUCCESS; }
int MPI_Comm_free(MPI_Comm* c) { if (*c > 1) g_comms.erase(*c); *c = MPI_COMM_NULL; return MPI_SUCCESS; }

int MPI_Send(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    std::vector<char> tmp; size_t bytes;
    const void* p = pack(buf, count, t, tmp, &bytes);
    raw_send(c.world.at(dest), c.ctx, tag, p, bytes);
    return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int src, int tag, MPI_Comm comm, MPI_Request* rq) {
    Comm& c = comm_of(comm);
    Req* q = raw_irecv(c.world.at(src), c.ctx, tag, buf, (size_t)count * type_size(t));
    int id = g_next_req++; g_reqs[id] = q; *rq = id;
    return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* rq, MPI_Status*) {
    if (*rq == MPI_REQUEST_NULL) return MPI_SUCCESS;
    auto it = g_reqs.find(*rq);
    if (it == g_reqs.end()) die("invalid request");
    raw_wait(it->second); g_reqs.erase(it); *rq = MPI_REQUEST_NULL;
    return MPI_SUCCESS;
}
int MPI_Waitall(int n, MPI_Request* rq, MPI_Status*) { for (int i = 0; i < n; ++i) MPI_Wait(&rq[i], nullptr); return MPI_SUCCESS; }
int MPI_Recv(void* buf, int count, MPI_Datatype t, int src, int tag, MPI_Comm comm, MPI_Status*) {
    Comm& c = comm_of(comm);
    raw_recv(c.world.at(src), c.ctx, tag, buf, (size_t)count * type_size(t));
    return MPI_SUCCESS;
}

int MPI_Barrier(MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const int n = (int)c.world.size(); char b = 0;
    if (c.myrank == 0) {
        for (int i = 1; i < n; ++i) raw_recv(c.world[i], c.ctx, TAG_COLL - 1, &b, 1);
        for (int i = 1; i < n; ++i) raw_send(c.world[i], c.ctx, TAG_COLL - 2, &b, 1);
    } else {
        raw_send(c.world[0], c.ctx, TAG_COLL - 1, &b, 1);
        raw_recv(c.world[0], c.ctx, TAG_COLL - 2, &b, 1);
    }
    return MPI_SUCCESS;
}

int MPI_Bcast(void* buf, int count, MPI_Datatype t, int root, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const size_t bytes = (size_t)count * type_size(t);
    const int n = (int)c.world.size();
    if (c.myrank == root) { for (int i = 0; i < n; ++i) if (i != root) raw_send(c.world[i], c.ctx, TAG_COLL - 3, buf, bytes); }
    else raw_recv(c.world[root], c.ctx, TAG_COLL - 3, buf, bytes);
    return MPI_SUCCESS;
}
int MPI_Ibcast(void* buf, int count, MPI_Datatype t, int root, MPI_Comm comm, MPI_Request* rq) {
    MPI_Bcast(buf, count, t, root, comm); *rq = MPI_REQUEST_NULL; return MPI_SUCCESS;
}

int MPI_Reduce(const void* s, void* r, int count, MPI_Datatype t, MPI_Op op, int root, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const size_t bytes = (size_t)count * type_size(t);
    const int n = (int)c.world.size();
    if (c.myrank != root) { raw_send(c.world[root], c.ctx, TAG_COLL - 4, s == MPI_IN_PLACE ? r : s, bytes); return MPI_SUCCESS; }
    std::vector<char> tmp(bytes), acc(bytes);
    // accumulate in rank order so that results do not depend on arrival order
    for (int i = 0; i < n; ++i) {
        const void* src;
        if (i == root) src = (s == MPI_IN_PLACE) ? r : s;
        else { raw_recv(c.world[i], c.ctx, TAG_COLL - 4, tmp.data(), bytes); src = tmp.data(); }
        if (i == 0) memcpy(acc.data(), src, bytes); else reduce_into(acc.data(), src, count, t, op);
    }
    memcpy(r, acc.data(), bytes);
    return MPI_SUCCESS;
}
int MPI_Allreduce(const void* s, void* r, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm) {
    MPI_Reduce(s, r, count, t, op, 0, comm);
    return MPI_Bcast(r, count, t, 0, comm);
}
int MPI_Reduce_scatter(const void* s, void* r, const int* counts, MPI_Datatype t, MPI_Op op, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const int n = (int)c.world.size();
    const size_t es = type_size(t);
    std::vector<size_t> off(n + 1, 0);
    for (int i = 0; i < n; ++i) off[i + 1] = off[i] + (size_t)counts[i];
    const size_t mine = (size_t)counts[c.myrank] * es;
    // pairwise exchange: slice j of every rank goes to rank j, which adds them in rank order
    std::vector<std::vector<char>> in(n);
    std::vector<Req*> reqs(n, nullptr);
    for (int i = 0; i < n; ++i) if (i != c.myrank) { in[i].resize(mine); reqs[i] = raw_irecv(c.world[i], c.ctx, TAG_COLL - 5, in[i].data(), mine); }
    for (int k = 1; k < n; ++k) { int j = (c.myrank + k) % n; raw_send(c.world[j], c.ctx, TAG_COLL - 5, (const char*)s + off[j] * es, (size_t)counts[j] * es); }
    std::vector<char> acc(mine);
    for (int i = 0; i < n; ++i) {
        const void* src;
        if (i == c.myrank) src = (const char*)s + off[i] * es; else { raw_wait(reqs[i]); src = in[i].data(); }
        if (i == 0) memcpy(acc.data(), src, mine); else reduce_into(acc.data(), src, counts[c.myrank], t, op);
    }
    memcpy(r, acc.data(), mine);
    return MPI_SUCCESS;
}

int MPI_Alltoallv(const void* s, const int* sc, const int* sd, MPI_Datatype st, void* r, const int* rc,
                  const int* rd, MPI_Datatype rt, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const int n = (int)c.world.size();
    const size_t ss = type_size(st), rs = type_size(rt);
    std::vector<Req*> reqs(n, nullptr);
    for (int i = 0; i < n; ++i) if (i != c.myrank) reqs[i] = raw_irecv(c.world[i], c.ctx, TAG_COLL - 6, (char*)r + (size_t)rd[i] * rs, (size_t)rc[i] * rs);
    memcpy((char*)r + (size_t)rd[c.myrank] * rs, (const char*)s + (size_t)sd[c.myrank] * ss, (size_t)sc[c.myrank] * ss);
    for (int k = 1; k < n; ++k) { int j = (c.myrank + k) % n; raw_send(c.world[j], c.ctx, TAG_COLL - 6, (const char*)s + (size_t)sd[j] * ss, (size_t)sc[j] * ss); }
    for (int i = 0; i < n; ++i) if (reqs[i]) raw_wait(reqs[i]);
    return MPI_SUCCESS;
}
int MPI_Alltoall(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm) {
    int n; MPI_Comm_size(comm, &n);
    std::vector<int> scv(n, sc), rcv(n, rc), sd(n), rd(n);
    for (int i = 0; i < n; ++i) { sd[i] = i * sc; rd[i] = i * rc; }
    return MPI_Alltoallv(s, scv.data(), sd.data(), st, r, rcv.data(), rd.data(), rt, comm);
}
int MPI_Allgatherv(const void* s, int sc, MPI_Datatype st, void* r, const int* rc, const int* rd, MPI_Datatype rt, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const int n = (int)c.world.size();
    const size_t ss = type_size(st), rs = type_size(rt);
    std::vector<Req*> reqs(n, nullptr);
    for (int i = 0; i < n; ++i) if (i != c.myrank) reqs[i] = raw_irecv(c.world[i], c.ctx, TAG_COLL - 7, (char*)r + (size_t)rd[i] * rs, (size_t)rc[i] * rs);
    memcpy((char*)r + (size_t)rd[c.myrank] * rs, s, (size_t)sc * ss);
    for (int k = 1; k < n; ++k) { int j = (c.myrank + k) % n; raw_send(c.world[j], c.ctx, TAG_COLL - 7, s, (size_t)sc * ss); }
    for (int i = 0; i < n; ++i) if (reqs[i]) raw_wait(reqs[i]);
    return MPI_SUCCESS;
}

int MPI_Dist_graph_create_adjacent(MPI_Comm comm, int indeg, const int* srcs, const int*, int outdeg, const int* dsts,
                                   const int*, MPI_Info, int, MPI_Comm* out) {
    Comm& p = comm_of(comm);
    Comm c = p;
    c.ctx = mix(p.ctx * 1315423911ull + (++p.children) * 2654435761ull + 7);
    c.nb_in.assign(srcs, srcs + indeg); c.nb_out.assign(dsts, dsts + outdeg); c.children = 0;
    *out = new_comm(std::move(c));
    return MPI_SUCCESS;
}
int MPI_Neighbor_alltoallv(const void* s, const int* sc, const int* sd, MPI_Datatype st, void* r, const int* rc,
                           const int* rd, MPI_Datatype rt, MPI_Comm comm) {
    Comm& c = comm_of(comm);
    const size_t ss = type_size(st), rs = type_size(rt);
    std::vector<Req*> reqs;
    for (size_t i = 0; i < c.nb_in.size(); ++i) reqs.push_back(raw_irecv(c.world[c.nb_in[i]], c.ctx, TAG_COLL - 8, (char*)r + (size_t)rd[i] * rs, (size_t)rc[i] * rs));
    for (size_t i = 0; i < c.nb_out.size(); ++i) raw_send(c.world[c.nb_out[i]], c.ctx, TAG_COLL - 8, (const char*)s + (size_t)sd[i] * ss, (size_t)sc[i] * ss);
    for (auto q : reqs) raw_wait(q);
    return MPI_SUCCESS;
}

// ---- Cartesian topologies ----------------------------------------------------
int MPI_Dims_create(int nnodes, int ndims, int* dims) {
    int fixed = 1, nfree = 0;
    for (int i = 0; i < ndims; ++i) { if (dims[i] > 0) fixed *= dims[i]; else ++nfree; }
    if (fixed <= 0 || nnodes % fixed) die("MPI_Dims_create: fixed dims do not divide the node count");
    int rest = nnodes / fixed;
    // prime factors, largest first, each given to the currently smallest free dimension
    std::vector<int> f;
    for (int p = 2; p * p <= rest; ++p) while (rest % p == 0) { f.push_back(p); rest /= p; }
    if (rest > 1) f.push_back(rest);
    std::sort(f.rbegin(), f.rend());
    std::vector<int> fr(nfree, 1);
    for (int p : f) { *std::min_element(fr.begin(), fr.end()) *= p; }
    std::sort(fr.rbegin(), fr.rend());
    for (int i = 0, k = 0; i < ndims; ++i) if (dims[i] <= 0) dims[i] = fr[k++];
    return MPI_SUCCESS;
}
int MPI_Cart_create(MPI_Comm comm, int ndims, const int* dims, const int*, int, MPI_Comm* out) {
    Comm& p = comm_of(comm);
    Comm c;
    c.ctx = mix(p.ctx * 1315423911ull + (++p.children) * 2654435761ull + 11);
    c.world = p.world; c.myrank = p.myrank; c.ndims = ndims; c.dims.assign(dims, dims + ndims);
    c.coords.resize(ndims);
    int rem = c.myrank;
    for (int d = ndims - 1; d >= 0; --d) { c.coords[d] = rem % dims[d]; rem /= dims[d]; }
    *out = new_comm(std::move(c));
    return MPI_SUCCESS;
}
int MPI_Cart_sub(MPI_Comm comm, const int* remain, MPI_Comm* out) {
    Comm& p = comm_of(comm);
    Comm c;
    uint64_t color = 0;
    for (int d = 0; d < p.ndims; ++d) if (!remain[d]) color = color * 100003 + p.coords[d] + 1;
    c.ctx = mix(p.ctx * 1315423911ull + (++p.children) * 2654435761ull + mix(color) + 13);
    for (int d = 0; d < p.ndims; ++d) if (remain[d]) { c.dims.push_back(p.dims[d]); c.coords.push_back(p.coords[d]); }
    c.ndims = (int)c.dims.size();
    const int n = (int)p.world.size();
    for (int r = 0; r < n; ++r) {  // members: same coordinates on the dropped dims, in parent rank order
        int rem = r; std::vector<int> co(p.ndims);
        for (int d = p.ndims - 1; d >= 0; --d) { co[d] = rem % p.dims[d]; rem /= p.dims[d]; }
        bool same = true;
        for (int d = 0; d < p.ndims; ++d) if (!remain[d] && co[d] != p.coords[d]) same = false;
        if (same) { if (r == p.myrank) c.myrank = (int)c.world.size(); c.world.push_back(p.world[r]); }
    }
    *out = new_comm(std::move(c));
    return MPI_SUCCESS;
}
int MPI_Cart_get(MPI_Comm comm, int maxdims, int* dims, int* periods, int* coords) {
    Comm& c = comm_of(comm);
    for (int d = 0; d < maxdims && d < c.ndims; ++d) { dims[d] = c.dims[d]; periods[d] = 0; coords[d] = c.coords[d]; }
    return MPI_SUCCESS;
}
int MPI_Cart_coords(MPI_Comm comm, int rank, int maxdims, int* coords) {
    Comm& c = comm_of(comm);
    std::vector<int> co(c.ndims);
    int rem = rank;
    for (int d = c.ndims - 1; d >= 0; --d) { co[d] = rem % c.dims[d]; rem /= c.dims[d]; }
    for (int d = 0; d < maxdims && d < c.ndims; ++d) coords[d] = co[d];
    return MPI_SUCCESS;
}
int MPI_Cart_rank(MPI_Comm comm, const int* coords, int* rank) {
    Comm& c = comm_of(comm);
    int r = 0;
    for (int d = 0; d < c.ndims; ++d) r = r * c.dims[d] + coords[d];
    *rank = r;
    return MPI_SUCCESS;
}

// ---- datatypes -----------------------------------------------------------------
int MPI_Type_create_struct(int n, const int* blens, const MPI_Aint* disps, const MPI_Datatype* types, MPI_Datatype* out) {
    DType d; size_t end = 0;
    for (int i = 0; i < n; ++i) end = std::max(end, (size_t)disps[i] + (size_t)blens[i] * type_size(types[i]));
    d.size = end;  // callers use structs without padding: treated as one contiguous blob
    int id = g_next_type++; g_types[id] = d; *out = id;
    return MPI_SUCCESS;
}
int MPI_Type_create_indexed_block(int n, int blen, const int* disps, MPI_Datatype old, MPI_Datatype* out) {
    DType d; const size_t es = type_size(old);
    for (int i = 0; i < n; ++i) d.blocks.push_back({(ptrdiff_t)disps[i] * (ptrdiff_t)es, (size_t)blen * es});
    d.size = (size_t)n * blen * es;
    int id = g_next_type++; g_types[id] = d; *out = id;
    return MPI_SUCCESS;
}
int MPI_Type_indexed(int n, const int* blens, const int* disps, MPI_Datatype old, MPI_Datatype* out) {
    DType d; const size_t es = type_size(old);
    for (int i = 0; i < n; ++i) { d.blocks.push_back({(ptrdiff_t)disps[i] * (ptrdiff_t)es, (size_t)blens[i] * es}); d.size += (size_t)blens[i] * es; }
    int id = g_next_type++; g_types[id] = d; *out = id;
    return MPI_SUCCESS;
}
int MPI_Type_commit(MPI_Datatype*) { return MPI_SUCCESS; }
int MPI_Type_free(MPI_Datatype* t) { g_types.erase(*t); *t = MPI_DATATYPE_NULL; return MPI_SUCCESS; }

// ---- file reads ------------------------------------------------------------------
int MPI_File_open(MPI_Comm, const char* name, int, MPI_Info, MPI_File* fh) {
    FILE* f = fopen(name, "rb");
    if (!f) die("MPI_File_open: cannot open file");
    setvbuf(f, nullptr, _IOFBF, 1 << 22);
    int id = g_next_file++; g_files[id] = f; *fh = id;
    return MPI_SUCCESS;
}
int MPI_File_read(MPI_File fh, void* buf, int count, MPI_Datatype t, MPI_Status*) {
    size_t bytes = (size_t)count * type_size(t);
    if (fread(buf, 1, bytes, g_files.at(fh)) != bytes) die("MPI_File_read: short read");
    return MPI_SUCCESS;
}
int MPI_File_seek(MPI_File fh, MPI_Offset off, int whence) {
    fseeko(g_files.at(fh), (off_t)off, whence == MPI_SEEK_CUR ? SEEK_CUR : SEEK_SET);
    return MPI_SUCCESS;
}
int MPI_File_close(MPI_File* fh) { fclose(g_files.at(*fh)); g_files.erase(*fh); *fh = 0; return MPI_SUCCESS; }

}  // extern "C"
