// Multi-GPU side of the path: partition arithmetic and the optional gather of the output shards, behind the C ABI.
//
// The quantised matmuls shard with no data-path collective (weight columns for the decode and per-block shapes, the batch
// axis for the batched MX shapes); the reference has no multi-device code for these operators. What a caller may still want
// is the whole output on every rank: one ncclAllGather of the shards over NVLink. Batch shards land in place (they are
// contiguous in the full output); column shards land rank-major in workspace and one small kernel interleaves them into
// rows. NCCL is not linked: its five entry points are resolved at run time from the libnccl.so.2 the process already
// carries (the one a PyTorch host loaded, or the system one), so the library loads on machines without it.
#include <dlfcn.h>

#include <atomic>
#include <cstdlib>

#include <map>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "opsnn_b200_shard.h"

namespace opsnn {

void set_err(const char* fmt, ...);

namespace {

struct NcclUniqueId {
    char internal[128];
};
using ncclComm_t = void*;
struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int /*ncclDataType_t*/, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

const NcclApi& nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString;
    });
    return api;
}

// One symmetric allocation: this rank's memory and the other ranks' memory of the same size, mapped here through CUDA IPC.
struct Symmetric {
    void* local = nullptr;
    uint64_t bytes = 0;
    std::vector<void*> peers;  // [world]; peers[rank] == local
};

struct Comm {
    ncclComm_t nccl = nullptr;
    int world = 1, rank = 0;
    std::vector<Symmetric> regions;
    // cross-rank arrival flags (a symmetric region of its own, made on first use): flags[r] = the last epoch rank r announced here
    Symmetric flags;
    unsigned int* done = nullptr;         // device ticket of the push kernel's CTAs (the last one to finish advances the epoch)
    unsigned long long* epoch = nullptr;  // device counter of this rank's arrivals: advanced by the kernel itself, so a captured launch replays correctly
    unsigned int* status = nullptr;       // device word: 0, or 1 when a wait for the other ranks ran out
};

std::mutex g_bind_mu;
std::map<const void*, PeerBinding> g_bindings;
std::atomic<int> g_binding_count{0};  // lets every decode launch skip the lock while nothing is bound

int32_t nccl_fail(const char* what, int rc)
{
    set_err("%s: NCCL error %d (%s)", what, rc, nccl().GetErrorString ? nccl().GetErrorString(rc) : "?");
    return (int32_t)cudaErrorUnknown;
}

// recv is [world][m][wmax] elements of `eb` bytes; rank r's block holds its columns [begin_r, end_r) in its first end_r - begin_r
// columns. 16-byte pieces when every width and the row pitch allow it, else bytes.
template <typename T>
__global__ void interleave_columns_kernel(const T* __restrict__ recv, T* __restrict__ full, int64_t m, int64_t n_total_t, int64_t wmax_t,
                                          int32_t world, int64_t units, int64_t mult_t)
{
    const int64_t base = units / world, extra = units % world;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < m * n_total_t; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / n_total_t, col = i - row * n_total_t;
        // owner of column `col`: the first `extra` ranks hold base + 1 units of `mult_t` columns, the others base; a ragged tail
        // shorter than one unit belongs to the last rank that owns anything
        int64_t u = col / mult_t;
        if (u >= units) u = units - 1;
        int64_t r = (u < extra * (base + 1)) ? u / (base + 1) : extra + (base > 0 ? (u - extra * (base + 1)) / base : 0);
        const int64_t begin = (r * base + (r < extra ? r : extra)) * mult_t;
        full[i] = recv[(r * m + row) * wmax_t + (col - begin)];
    }
}

// The same move in 16-byte pieces, one rank's run per blockIdx.y: in a row, rank r's columns are contiguous both in its receive
// block and in the full row. Needs every run to start and end on a 16-byte boundary in both places (checked on the host).
constexpr int kMaxRunRanks = 64;
struct ColumnRuns {
    int64_t begin_b[kMaxRunRanks];  // byte offset of the rank's first column in a full row
    int64_t width_b[kMaxRunRanks];  // bytes of a row the rank owns
};

__global__ void interleave_runs_kernel(const uint8_t* __restrict__ recv, uint8_t* __restrict__ full, int64_t m, int64_t full_row_b,
                                       int64_t block_row_b, const __grid_constant__ ColumnRuns runs)
{
    const int r = blockIdx.y;
    const int64_t pieces = runs.width_b[r] / 16, begin = runs.begin_b[r];
    const uint8_t* src = recv + (int64_t)r * m * block_row_b;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < m * pieces; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / pieces, p = i - row * pieces;
        *reinterpret_cast<uint4*>(full + row * full_row_b + begin + p * 16) = *reinterpret_cast<const uint4*>(src + row * block_row_b + p * 16);
    }
}

// Every rank writes its epoch into slot `rank` of every rank's flag array (release at system scope: the stores of the kernels
// before it in the stream are performed by then), then waits, bounded, until every slot of its own array holds the epoch.
struct FlagPeers {
    unsigned long long* flags[kMaxPeers];
};
__global__ void arrive_and_wait_kernel(const __grid_constant__ FlagPeers peers, int world, int rank, unsigned long long* epoch_counter,
                                       unsigned int limit, unsigned int* status)
{
    // Launched as a programmatic dependent of the kernel before it and a programmatic prerequisite of the one after: the next
    // kernel may be placed at once, and this one reads and writes nothing before the previous kernel has completed (its stores,
    // the peer stores included, are performed by then).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ unsigned long long s_epoch;
    if (threadIdx.x == 0) s_epoch = ++(*epoch_counter);  // every rank makes the same number of calls: the counters agree
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const int r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(peers.flags[r] + rank), "l"(epoch) : "memory");
    const unsigned long long* mine = peers.flags[rank] + r;
    bool seen = false;
    for (unsigned int i = 0; i < limit && !seen; ++i) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
        seen = v >= epoch;
        if (!seen) __nanosleep(100);
    }
    if (!seen) atomicExch(status, 1u);
}


// The all-gather of small column shards as one kernel over peer memory: the CTAs (blockIdx.x, r) copy this rank's (m, width)
// shard into rank r's full output (16-byte stores over NVLink, rows are contiguous on both sides); the last of them to finish
// (a ticket per peer) releases this rank's flag there and waits, bounded, for rank r's flag here. The epoch all CTAs use is the
// device counter + 1; the last of the `world` flag-handling CTAs to finish advances it.
struct PeerFull {
    uint8_t* full[kMaxPeers];
};
template <int VB>
__global__ void __launch_bounds__(256) allgather_columns_kernel(const __grid_constant__ FlagPeers flags, const __grid_constant__ PeerFull dst,
                                                                const uint8_t* __restrict__ y_local, int64_t local_row_b, int64_t width_b,
                                                                int64_t m, int64_t full_row_b, int64_t col0_b, int world, int rank,
                                                                unsigned long long* epoch_counter, unsigned int* done, unsigned int limit,
                                                                unsigned int* status)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the kernel that wrote y_local has completed
    const int r = blockIdx.y;
    const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(epoch_counter) + 1ull;
    uint8_t* out = dst.full[r] + col0_b;
    const int64_t pieces = width_b / VB;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < m * pieces; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / pieces, p = i - row * pieces;
        if (VB == 16)
            *reinterpret_cast<uint4*>(out + row * full_row_b + p * 16) = *reinterpret_cast<const uint4*>(y_local + row * local_row_b + p * 16);
        else
            *reinterpret_cast<uint16_t*>(out + row * full_row_b + p * 2) = *reinterpret_cast<const uint16_t*>(y_local + row * local_row_b + p * 2);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x != 0) return;
    // done[1 + r]: CTAs of peer r that have finished their part; done[0]: flag-handling CTAs that have finished
    if (atomicAdd(done + 1 + r, 1u) != gridDim.x - 1u) return;
    done[1 + r] = 0u;
    __threadfence_system();  // the other CTAs' stores (ordered before their tickets) before the flag
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flags.flags[r] + rank), "l"(epoch) : "memory");
    const unsigned long long* mine = flags.flags[rank] + r;
    bool seen = false;
    for (unsigned int i = 0; i < limit && !seen; ++i) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
        seen = v >= epoch;
        if (!seen) __nanosleep(100);
    }
    if (!seen) atomicExch(status, 1u);
    __threadfence();
    if (atomicAdd(done, 1u) == (unsigned int)world - 1u) {  // every CTA has read the counter long ago
        *done = 0u;
        *epoch_counter = epoch;
    }
}

}  // namespace

bool lookup_peer_binding(const void* y_local, PeerBinding* out)
{
    if (y_local == nullptr || g_binding_count.load(std::memory_order_acquire) == 0) return false;
    std::lock_guard<std::mutex> lk(g_bind_mu);
    auto it = g_bindings.find(y_local);
    if (it == g_bindings.end()) return false;
    *out = it->second;
    return true;
}

}  // namespace opsnn

using namespace opsnn;

namespace {

// Allocates `bytes` on every rank and maps every rank's block into this process (CUDA IPC; the handles travel through one
// ncclAllGather). Collective: every rank of the communicator calls it with the same size.
int32_t symmetric_alloc(Comm* c, uint64_t bytes, Symmetric* out)
{
    out->bytes = bytes;
    out->peers.assign((size_t)c->world, nullptr);
    cudaError_t rc = cudaMalloc(&out->local, bytes);
    if (rc != cudaSuccess) return (int32_t)rc;
    cudaMemset(out->local, 0, bytes);
    out->peers[(size_t)c->rank] = out->local;
    if (c->world == 1) return 0;
    cudaIpcMemHandle_t mine;
    rc = cudaIpcGetMemHandle(&mine, out->local);
    if (rc != cudaSuccess) return (int32_t)rc;
    uint8_t* dev = nullptr;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    rc = cudaMalloc(&dev, hb * (size_t)(c->world + 1));
    if (rc != cudaSuccess) return (int32_t)rc;
    cudaMemcpy(dev, &mine, hb, cudaMemcpyHostToDevice);
    const int nrc = nccl().AllGather(dev, dev + hb, hb, 0, c->nccl, (cudaStream_t)0);
    if (nrc != 0) {
        cudaFree(dev);
        return nccl_fail("ncclAllGather", nrc);
    }
    rc = cudaStreamSynchronize((cudaStream_t)0);
    std::vector<cudaIpcMemHandle_t> all((size_t)c->world);
    if (rc == cudaSuccess) rc = cudaMemcpy(all.data(), dev + hb, hb * (size_t)c->world, cudaMemcpyDeviceToHost);
    cudaFree(dev);
    if (rc != cudaSuccess) return (int32_t)rc;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        rc = cudaIpcOpenMemHandle(&out->peers[(size_t)r], all[(size_t)r], cudaIpcMemLazyEnablePeerAccess);
        if (rc != cudaSuccess) {
            set_err("opsnn_comm_symmetric_alloc: rank %d could not map rank %d's memory (CUDA error %d): the ranks must be processes of one node with peer access",
                    c->rank, r, (int)rc);
            return (int32_t)rc;
        }
    }
    return 0;
}

// The cross-rank flags and the device words beside them, made on first use (collective).
int32_t ensure_flags(Comm* c)
{
    if (c->flags.local != nullptr) return 0;
    const int32_t rc = symmetric_alloc(c, 256 * sizeof(unsigned long long), &c->flags);
    if (rc != 0) return rc;
    cudaError_t e = cudaMalloc(&c->status, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&c->epoch, sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(&c->done, 16 * sizeof(unsigned int));
    if (e != cudaSuccess) return (int32_t)e;
    cudaMemset(c->status, 0, sizeof(unsigned int));
    cudaMemset(c->epoch, 0, sizeof(unsigned long long));
    cudaMemset(c->done, 0, 16 * sizeof(unsigned int));
    cudaDeviceSynchronize();
    return 0;
}

void symmetric_release(Comm* c, Symmetric* sy)
{
    for (int r = 0; r < (int)sy->peers.size(); ++r)
        if (r != c->rank && sy->peers[(size_t)r] != nullptr) cudaIpcCloseMemHandle(sy->peers[(size_t)r]);
    if (sy->local != nullptr) cudaFree(sy->local);
    sy->local = nullptr;
    sy->peers.clear();
}

}  // namespace

extern "C" {

void opsnn_shard_range(int64_t total, int32_t world, int32_t rank, int64_t multiple, int64_t* begin, int64_t* end)
{
    int64_t b = 0, e = 0;
    if (world >= 1 && rank >= 0 && rank < world && total >= 0 && multiple >= 1) {
        const int64_t units = total / multiple, base = units / world, extra = units % world;
        const int64_t bu = rank * base + (rank < extra ? rank : extra);
        const int64_t eu = bu + base + (rank < extra ? 1 : 0);
        b = bu * multiple;
        e = eu * multiple;
        const int64_t tail = total - units * multiple;
        if (tail != 0) {
            const int64_t last_owner = units ? (world < units ? world : units) - 1 : 0;
            if (rank == last_owner) e += tail;
            if (units == 0 && rank != 0) b = e = total;
        }
    }
    if (begin) *begin = b;
    if (end) *end = e;
}

int32_t opsnn_comm_unique_id(void* id128)
{
    if (id128 == nullptr) return (int32_t)cudaErrorInvalidValue;
    if (!nccl().ok) {
        set_err("opsnn_comm_unique_id: libnccl.so.2 could not be loaded");
        return (int32_t)cudaErrorNotSupported;
    }
    const int rc = nccl().GetUniqueId(reinterpret_cast<NcclUniqueId*>(id128));
    return rc == 0 ? 0 : nccl_fail("ncclGetUniqueId", rc);
}

int32_t opsnn_comm_init(const void* id128, int32_t world, int32_t rank, void** comm)
{
    if (id128 == nullptr || comm == nullptr || world < 1 || rank < 0 || rank >= world) return (int32_t)cudaErrorInvalidValue;
    if (!nccl().ok) {
        set_err("opsnn_comm_init: libnccl.so.2 could not be loaded");
        return (int32_t)cudaErrorNotSupported;
    }
    Comm* c = new Comm();
    c->world = world;
    c->rank = rank;
    NcclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    const int rc = nccl().CommInitRank(&c->nccl, world, id, rank);
    if (rc != 0) {
        delete c;
        return nccl_fail("ncclCommInitRank", rc);
    }
    *comm = c;
    return 0;
}

int32_t opsnn_comm_destroy(void* comm)
{
    if (comm == nullptr) return 0;
    Comm* c = static_cast<Comm*>(comm);
    cudaDeviceSynchronize();
    {   // bindings into this communicator's symmetric memory go with it
        std::lock_guard<std::mutex> lk(g_bind_mu);
        for (auto it = g_bindings.begin(); it != g_bindings.end();) {
            bool ours = false;
            for (const Symmetric& sy : c->regions)
                for (void* q : sy.peers) ours = ours || q == it->second.full[0];
            it = ours ? g_bindings.erase(it) : std::next(it);
        }
        g_binding_count.store((int)g_bindings.size(), std::memory_order_release);
    }
    for (Symmetric& sy : c->regions) symmetric_release(c, &sy);
    c->regions.clear();
    if (c->flags.local != nullptr) symmetric_release(c, &c->flags);
    if (c->status != nullptr) cudaFree(c->status);
    if (c->epoch != nullptr) cudaFree(c->epoch);
    if (c->done != nullptr) cudaFree(c->done);
    const int rc = c->nccl ? nccl().CommDestroy(c->nccl) : 0;
    delete c;
    return rc == 0 ? 0 : nccl_fail("ncclCommDestroy", rc);
}

uint64_t opsnn_gather_columns_workspace(int32_t world, int64_t m, int64_t n_total, int64_t multiple, int32_t elem_bytes)
{
    int64_t wmax = 0;
    for (int32_t r = 0; r < world; ++r) {
        int64_t b, e;
        opsnn_shard_range(n_total, world, r, multiple, &b, &e);
        if (e - b > wmax) wmax = e - b;
    }
    // the padded send block of this rank + the rank-major receive area
    return (uint64_t)(world + 1) * (uint64_t)m * (uint64_t)wmax * (uint64_t)elem_bytes + 512;
}

int32_t opsnn_gather_columns(void* comm, const void* y_local, int64_t y_local_ld, int64_t m, int64_t n_total, int64_t multiple,
                             int32_t elem_bytes, void* y_full, void* workspace, uint64_t workspace_size, void* stream)
{
    if (comm == nullptr || y_local == nullptr || y_full == nullptr || m < 0 || n_total < 0 || multiple < 1 ||
        (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4))
        return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m == 0 || n_total == 0) return 0;
    int64_t wmax = 0, mine_b = 0, mine_e = 0;
    for (int32_t r = 0; r < c->world; ++r) {
        int64_t b, e;
        opsnn_shard_range(n_total, c->world, r, multiple, &b, &e);
        if (e - b > wmax) wmax = e - b;
        if (r == c->rank) mine_b = b, mine_e = e;
    }
    if (workspace == nullptr || workspace_size < opsnn_gather_columns_workspace(c->world, m, n_total, multiple, elem_bytes)) {
        set_err("opsnn_gather_columns: workspace of %llu bytes needed", (unsigned long long)opsnn_gather_columns_workspace(c->world, m, n_total, multiple, elem_bytes));
        return (int32_t)cudaErrorInvalidValue;
    }
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
    const size_t block = (size_t)m * (size_t)wmax * (size_t)elem_bytes;
    const uint8_t* send = ws;
    uint8_t* recv = ws + block;
    if (mine_e - mine_b == wmax && y_local_ld == wmax) {
        send = static_cast<const uint8_t*>(y_local);  // the shard already is a dense (m, wmax) block: sent from where it lies
    } else {
        // this rank's (m, width) shard into the head of a (m, wmax) block: one strided copy on the stream
        cudaError_t rc = cudaMemcpy2DAsync(ws, (size_t)wmax * elem_bytes, y_local, (size_t)y_local_ld * elem_bytes,
                                           (size_t)(mine_e - mine_b) * elem_bytes, (size_t)m, cudaMemcpyDeviceToDevice, s);
        if (rc != cudaSuccess) return (int32_t)rc;
    }
    const int nrc = nccl().AllGather(send, recv, block, 0 /* ncclInt8: the payload is moved as bytes */, c->nccl, s);
    if (nrc != 0) return nccl_fail("ncclAllGather", nrc);
    const int64_t units = n_total / multiple;
    const int64_t total = m * n_total;
    const int threads = 256;
    // 16-byte pieces when every rank's run starts and ends on a 16-byte boundary of the full row and of its receive block
    ColumnRuns runs{};
    bool vec = c->world <= kMaxRunRanks && (reinterpret_cast<uintptr_t>(y_full) % 16) == 0 && ((size_t)n_total * elem_bytes) % 16 == 0 &&
               ((size_t)wmax * elem_bytes) % 16 == 0;
    for (int32_t r = 0; vec && r < c->world; ++r) {
        int64_t b, e;
        opsnn_shard_range(n_total, c->world, r, multiple, &b, &e);
        runs.begin_b[r] = b * elem_bytes;
        runs.width_b[r] = (e - b) * elem_bytes;
        vec = runs.begin_b[r] % 16 == 0 && runs.width_b[r] % 16 == 0;
    }
    if (vec) {
        const int64_t per_rank = m * ((int64_t)wmax * elem_bytes / 16);
        const int bx = (int)((per_rank + threads - 1) / threads < 296 ? (per_rank + threads - 1) / threads : 296);
        interleave_runs_kernel<<<dim3((unsigned)(bx < 1 ? 1 : bx), (unsigned)c->world, 1), threads, 0, s>>>(
            recv, static_cast<uint8_t*>(y_full), m, n_total * elem_bytes, wmax * elem_bytes, runs);
        note_launch("gather_interleave");
        return (int32_t)cudaGetLastError();
    }
    const int blocks = (int)((total + threads - 1) / threads < 1184 ? (total + threads - 1) / threads : 1184);
    if (elem_bytes == 2)
        interleave_columns_kernel<uint16_t><<<blocks, threads, 0, s>>>(reinterpret_cast<const uint16_t*>(recv), static_cast<uint16_t*>(y_full), m, n_total,
                                                                     wmax, c->world, units, multiple);
    else if (elem_bytes == 4)
        interleave_columns_kernel<uint32_t><<<blocks, threads, 0, s>>>(reinterpret_cast<const uint32_t*>(recv), static_cast<uint32_t*>(y_full), m, n_total,
                                                                     wmax, c->world, units, multiple);
    else
        interleave_columns_kernel<uint8_t><<<blocks, threads, 0, s>>>(recv, static_cast<uint8_t*>(y_full), m, n_total, wmax, c->world, units, multiple);
    note_launch("gather_interleave");
    return (int32_t)cudaGetLastError();
}

int32_t opsnn_gather_batch(void* comm, const void* y_local, int64_t batch_total, uint64_t bytes_per_batch, void* y_full, void* stream)
{
    if (comm == nullptr || y_local == nullptr || y_full == nullptr || batch_total < 0) return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    if (batch_total % c->world != 0) {
        set_err("opsnn_gather_batch: %lld batches do not divide over %d ranks (ncclAllGather moves equal shares)", (long long)batch_total, c->world);
        return (int32_t)cudaErrorInvalidValue;
    }
    if (batch_total == 0 || bytes_per_batch == 0) return 0;
    const size_t share = (size_t)(batch_total / c->world) * (size_t)bytes_per_batch;
    // in place when the caller's shard already sits at its slot of y_full (NCCL's in-place rule), else from y_local
    const int nrc = nccl().AllGather(y_local, y_full, share, 0, c->nccl, static_cast<cudaStream_t>(stream));
    return nrc == 0 ? 0 : nccl_fail("ncclAllGather", nrc);
}


int32_t opsnn_comm_symmetric_alloc(void* comm, uint64_t bytes, void** local, void** peers)
{
    if (comm == nullptr || local == nullptr || bytes == 0) return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    if (c->world > kMaxPeers) {
        set_err("opsnn_comm_symmetric_alloc: at most %d ranks", kMaxPeers);
        return (int32_t)cudaErrorNotSupported;
    }
    Symmetric sy;
    const int32_t rc = symmetric_alloc(c, bytes, &sy);
    if (rc != 0) {
        symmetric_release(c, &sy);
        return rc;
    }
    *local = sy.local;
    if (peers != nullptr)
        for (int r = 0; r < c->world; ++r) peers[r] = sy.peers[(size_t)r];
    c->regions.push_back(sy);
    return 0;
}

int32_t opsnn_comm_symmetric_free(void* comm, void* local)
{
    if (comm == nullptr || local == nullptr) return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    for (size_t i = 0; i < c->regions.size(); ++i) {
        if (c->regions[i].local != local) continue;
        cudaDeviceSynchronize();
        symmetric_release(c, &c->regions[i]);
        c->regions.erase(c->regions.begin() + (long)i);
        return 0;
    }
    return (int32_t)cudaErrorInvalidValue;
}

int32_t opsnn_comm_bind_columns(void* comm, const void* y_local, const void* y_full_local, int64_t n_total, int64_t multiple)
{
    if (comm == nullptr || y_local == nullptr || y_full_local == nullptr || n_total < 1 || multiple < 1) return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    const Symmetric* sy = nullptr;
    for (const Symmetric& s : c->regions)
        if (s.local == y_full_local) sy = &s;
    if (sy == nullptr) {
        set_err("opsnn_comm_bind_columns: y_full was not allocated by opsnn_comm_symmetric_alloc on this communicator");
        return (int32_t)cudaErrorInvalidValue;
    }
    PeerBinding b{};
    b.count = c->world;
    for (int r = 0; r < c->world; ++r) b.full[r] = sy->peers[(size_t)r];
    b.ld = n_total;
    int64_t begin = 0, end = 0;
    opsnn_shard_range(n_total, c->world, c->rank, multiple, &begin, &end);
    b.col0 = begin;
    std::lock_guard<std::mutex> lk(g_bind_mu);
    g_bindings[y_local] = b;
    g_binding_count.store((int)g_bindings.size(), std::memory_order_release);
    return 0;
}

int32_t opsnn_comm_unbind(const void* y_local)
{
    std::lock_guard<std::mutex> lk(g_bind_mu);
    g_bindings.erase(y_local);
    g_binding_count.store((int)g_bindings.size(), std::memory_order_release);
    return 0;
}

int32_t opsnn_comm_arrive_and_wait(void* comm, void* stream)
{
    if (comm == nullptr) return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    if (c->world > kMaxPeers) return (int32_t)cudaErrorNotSupported;
    if (const int32_t rc = ensure_flags(c)) return rc;
    FlagPeers fp{};
    for (int r = 0; r < c->world; ++r) fp.flags[r] = static_cast<unsigned long long*>(c->flags.peers[(size_t)r]);
    // about a second of polling at 100 ns per poll before the wait is declared dead
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(32, 1, 1);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    unsigned int limit = 4u * 1000u * 1000u;
    if (const char* e = getenv("OPSNN_COMM_POLL_LIMIT")) {  // tests of the give-up path: a shorter wait
        const long v = atol(e);
        if (v > 0 && v < (long)limit) limit = (unsigned int)v;
    }
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, arrive_and_wait_kernel, fp, c->world, c->rank, c->epoch, limit, c->status);
    note_launch("comm_arrive_and_wait");
    return (int32_t)rc;
}

uint32_t opsnn_comm_status(void* comm, int32_t reset)
{
    if (comm == nullptr) return 0;
    Comm* c = static_cast<Comm*>(comm);
    if (c->status == nullptr) return 0;
    unsigned int v = 0;
    cudaMemcpy(&v, c->status, sizeof(v), cudaMemcpyDeviceToHost);
    if (reset) cudaMemset(c->status, 0, sizeof(unsigned int));
    return v;
}


int32_t opsnn_comm_allgather_columns(void* comm, const void* y_local, int64_t y_local_ld, int64_t m, const void* y_full_local, int64_t n_total,
                                     int64_t multiple, int32_t elem_bytes, void* stream)
{
    if (comm == nullptr || y_local == nullptr || y_full_local == nullptr || m < 0 || n_total < 1 || multiple < 1 ||
        (elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 1))
        return (int32_t)cudaErrorInvalidValue;
    Comm* c = static_cast<Comm*>(comm);
    if (c->world > kMaxPeers) return (int32_t)cudaErrorNotSupported;
    const Symmetric* sy = nullptr;
    for (const Symmetric& s : c->regions)
        if (s.local == y_full_local) sy = &s;
    if (sy == nullptr) {
        set_err("opsnn_comm_allgather_columns: y_full was not allocated by opsnn_comm_symmetric_alloc on this communicator");
        return (int32_t)cudaErrorInvalidValue;
    }
    if (const int32_t rc = ensure_flags(c)) return rc;
    int64_t begin = 0, end = 0;
    opsnn_shard_range(n_total, c->world, c->rank, multiple, &begin, &end);
    FlagPeers fp{};
    PeerFull pf{};
    for (int r = 0; r < c->world; ++r) {
        fp.flags[r] = static_cast<unsigned long long*>(c->flags.peers[(size_t)r]);
        pf.full[r] = static_cast<uint8_t*>(sy->peers[(size_t)r]);
    }
    const int64_t width_b = (end - begin) * elem_bytes, col0_b = begin * elem_bytes, full_row_b = n_total * elem_bytes, local_row_b = y_local_ld * elem_bytes;
    const bool vec = width_b % 16 == 0 && col0_b % 16 == 0 && full_row_b % 16 == 0 && local_row_b % 16 == 0 &&
                     (reinterpret_cast<uintptr_t>(y_local) & 15) == 0;
    if (!vec && (elem_bytes != 2 || width_b % 2 != 0)) {
        set_err("opsnn_comm_allgather_columns: shards that are not whole 16-byte pieces are moved as 2-byte elements only");
        return (int32_t)cudaErrorNotSupported;
    }
    unsigned int limit = 4u * 1000u * 1000u;
    if (const char* e = getenv("OPSNN_COMM_POLL_LIMIT")) {
        const long v = atol(e);
        if (v > 0 && v < (long)limit) limit = (unsigned int)v;
    }
    cudaLaunchConfig_t cfg{};
    // enough CTAs per peer that a copy is a handful of independent 16-byte round trips per thread, about 128 CTAs in all
    int64_t parts = 128 / c->world;
    const int64_t work = (m * (width_b / (vec ? 16 : 2)) + 255) / 256;
    if (parts > work) parts = work;
    if (parts < 1) parts = 1;
    cfg.gridDim = dim3((unsigned)parts, (unsigned)c->world, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const uint8_t* src = static_cast<const uint8_t*>(y_local);
    cudaError_t rc;
    if (vec)
        rc = cudaLaunchKernelEx(&cfg, allgather_columns_kernel<16>, fp, pf, src, local_row_b, width_b, m, full_row_b, col0_b, c->world, c->rank, c->epoch,
                                c->done, limit, c->status);
    else
        rc = cudaLaunchKernelEx(&cfg, allgather_columns_kernel<2>, fp, pf, src, local_row_b, width_b, m, full_row_b, col0_b, c->world, c->rank, c->epoch,
                                c->done, limit, c->status);
    note_launch("comm_allgather_columns");
    return (int32_t)rc;
}

}  // extern "C"
