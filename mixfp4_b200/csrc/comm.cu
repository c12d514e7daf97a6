// Peer-memory exchange area for the fused row-parallel GEMV + all-reduce (gemv.cu).
//
// Every rank (one process per GPU of one node) owns a receive buffer of 8-byte packets
// {fp32 partial sum, flag}: [2 parities][world source ranks][slot packets].  A rank's kernel
// stores its partial sums straight into every peer's buffer (plain 8-byte stores through the
// peer mapping, no multimem, no TMA) and polls its own buffer; the flag inside each packet is
// the launch's sequence number, so a packet validates itself and no fence or separate signal
// is needed.  The buffers are exported with cudaIpcGetMemHandle and opened by the peers; the
// handles travel through whatever the host uses for rendezvous (torch.distributed in the
// Python wrapper).
//
// The two parities alternate between launches.  A rank can only finish launch e after every
// peer has started launch e (it needs their packets), and a peer starts launch e only after
// it has finished reading launch e-1, so when a rank starts writing launch e+1 into the
// parity of launch e-1 nobody reads that parity any more.

#include <new>

#include "common.cuh"

struct mixfp4_comm {
    int rank, world, device;
    int64_t slot_packets;
    uint2* recv;                 // this rank's buffer (device memory of this GPU)
    uint2* peer[8];              // every rank's buffer as seen from this GPU (peer[rank] == recv)
    uint32_t* words;             // [0] sequence number of the next launch, [1] finished-CTA counter
    bool opened;
    bool local;                  // peers are plain pointers of this process (mixfp4_comm_open_local)
};

using namespace mixfp4;

extern "C" int mixfp4_comm_create(int rank, int world, int64_t slot_floats, mixfp4_comm** out) {
    if (!out) return MIXFP4_E_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || slot_floats <= 0) return MIXFP4_E_SHAPE;
    mixfp4_comm* c = new (std::nothrow) mixfp4_comm();
    if (!c) return MIXFP4_E_CUDA;
    c->rank = rank; c->world = world; c->slot_packets = slot_floats; c->opened = world == 1; c->local = false;
    for (int i = 0; i < 8; ++i) c->peer[i] = nullptr;
    const size_t bytes = (size_t)2 * world * slot_floats * sizeof(uint2);
    cudaError_t err = cudaGetDevice(&c->device);
    if (err == cudaSuccess) err = cudaMalloc(&c->recv, bytes);
    if (err == cudaSuccess) err = cudaMemset(c->recv, 0, bytes);
    if (err == cudaSuccess) err = cudaMalloc(&c->words, 2 * sizeof(uint32_t));
    if (err == cudaSuccess) err = cudaMemset(c->words, 0, 2 * sizeof(uint32_t));
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        if (c->recv) cudaFree(c->recv);
        if (c->words) cudaFree(c->words);
        delete c;
        return record_cuda_error(err, "mixfp4_comm_create");
    }
    c->peer[rank] = c->recv;
    *out = c;
    return MIXFP4_OK;
}

extern "C" int mixfp4_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int mixfp4_comm_handle(const mixfp4_comm* c, void* handle) {
    if (!c || !handle) return MIXFP4_E_NULL;
    cudaIpcMemHandle_t h;
    MIXFP4_CUDA_CHECK(cudaIpcGetMemHandle(&h, c->recv));
    memcpy(handle, &h, sizeof(h));
    return MIXFP4_OK;
}

// handles: world consecutive handles in rank order (this rank's own entry is ignored).
extern "C" int mixfp4_comm_open(mixfp4_comm* c, const void* handles) {
    if (!c || !handles) return MIXFP4_E_NULL;
    if (c->opened) return MIXFP4_OK;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        MIXFP4_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->peer[r] = static_cast<uint2*>(p);
    }
    c->opened = true;
    return MIXFP4_OK;
}

extern "C" int64_t mixfp4_comm_buffer_bytes(int world, int64_t slot_floats) {
    return world >= 1 && world <= 8 && slot_floats > 0 ? (int64_t)2 * world * slot_floats * (int64_t)sizeof(uint2) : 0;
}

extern "C" int mixfp4_comm_buffer(const mixfp4_comm* c, void** buffer) {
    if (!c || !buffer) return MIXFP4_E_NULL;
    *buffer = c->recv;
    return MIXFP4_OK;
}

extern "C" int mixfp4_comm_open_local(mixfp4_comm* c, void* const* buffers) {
    if (!c || !buffers) return MIXFP4_E_NULL;
    if (c->opened) return MIXFP4_OK;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        if (!buffers[r]) return MIXFP4_E_NULL;
        if (!aligned(buffers[r], 8)) return MIXFP4_E_ALIGN;
        c->peer[r] = static_cast<uint2*>(buffers[r]);
    }
    c->opened = true;
    c->local = true;
    return MIXFP4_OK;
}

extern "C" int mixfp4_comm_destroy(mixfp4_comm* c) {
    if (!c) return MIXFP4_OK;
    for (int r = 0; r < c->world; ++r)
        if (!c->local && r != c->rank && c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
    cudaFree(c->recv);
    cudaFree(c->words);
    delete c;
    return MIXFP4_OK;
}

namespace mixfp4 {
// For gemv.cu: the pieces of a communicator the kernel needs.
int comm_view(const mixfp4_comm* c, int* rank, int* world, int64_t* slot_packets, uint2** recv, uint2** peers,
              uint32_t** words) {
    if (!c) return MIXFP4_E_NULL;
    if (!c->opened) return MIXFP4_E_MODE;
    *rank = c->rank; *world = c->world; *slot_packets = c->slot_packets; *recv = c->recv; *words = c->words;
    for (int i = 0; i < 8; ++i) peers[i] = c->peer[i];
    return MIXFP4_OK;
}
}  // namespace mixfp4
