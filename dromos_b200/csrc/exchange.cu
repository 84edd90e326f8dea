// The exchange step of a row-sharded product as ONE kernel over peer-mapped memory: every rank has written its slice
// of y (its columns of the whole [M, ld_y] output) into its own copy of the whole y; this kernel stores that slice into
// every other rank's copy (plain NVLink stores, 16 bytes per thread where the slice allows), tells every rank's arrival
// semaphore once, and waits (bounded) until its own semaphore holds one arrival per rank, which it takes. When the
// kernel is done, this rank's y is whole. No collective library runs and nothing is staged: at decode sizes (a few KB
// to 1 MB per rank) an NCCL all-gather costs 17-37 us per product on 2-8 GPUs, of which the bytes are 1-2 us.
//
// The semaphores count: arrivals of the next round that come early stay in the counter, and nothing depends on how often
// the call has run, so the call can sit in a replayed graph. Peers must not be more than one round ahead of a rank
// that still reads y: callers alternate two y buffers.
#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kStatusExchangeWait = 6;  // the wait for the peers' slices gave up

struct ExchangeParams {
  uint8_t* y[kMaxRanks];     // every rank's whole y (peer-mapped), already offset to this rank's first column
  int* arrive[kMaxRanks];    // every rank's arrival semaphore (word 0 of its counter pair)
  int* done_local;           // this rank's count of finished CTAs (word 1 of its own counter pair)
  int ranks, self, M;
  int64_t row_bytes;         // bytes of a slice row
  int64_t pitch;             // bytes between rows of the whole y
  int* status;
  uint64_t budget_ns;
};

template <int V>  // bytes per thread and store: 16, 4 or 2
__global__ void __launch_bounds__(256) exchange_kernel(const ExchangeParams P) {
  pdl_trigger();
  pdl_wait();  // the slice comes from the product before this kernel
  // One (peer, piece of the slice) pair per thread and turn, pieces fastest: a warp stores 512 contiguous bytes to one peer,
  // the warps of the grid cover all peers at once, and the grid grows with the number of peers (with a thread storing its piece to every peer in turn, 56 CTAs carried the
  // 6.4 MB a rank sends at M = 64 on 8 GPUs, and the exchange took 35 us).
  const int64_t per_row = P.row_bytes / V, pieces = per_row * P.M;
  const int peers = P.ranks - 1;
  const int64_t total = pieces * peers;
  const uint8_t* src = P.y[P.self];
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < total; j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int r = static_cast<int>(j / pieces);
    const int64_t i = j - r * pieces;
    r += r >= P.self;  // skip this rank
    const int64_t m = i / per_row, at = m * P.pitch + (i - m * per_row) * V;
    if constexpr (V == 16) *reinterpret_cast<uint4*>(P.y[r] + at) = *reinterpret_cast<const uint4*>(src + at);
    else if constexpr (V == 4) *reinterpret_cast<uint32_t*>(P.y[r] + at) = *reinterpret_cast<const uint32_t*>(src + at);
    else *reinterpret_cast<uint16_t*>(P.y[r] + at) = *reinterpret_cast<const uint16_t*>(src + at);
  }
  // The CTA's stores are visible system-wide before it counts itself; the grid's last CTA tells every rank (one remote
  // atomic per rank and launch: atomics on one word serialise) and then waits for the peers.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  int before;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(P.done_local) : "memory");
  if (before != static_cast<int>(gridDim.x) - 1) return;
  asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(P.done_local), "r"(0) : "memory");
  __threadfence_system();
  // (relaxed: the fence above already orders this rank's stores before them; a release on each would wait for the one
  // before it, one NVLink round trip per rank: 23 us for a 14 KB slice on 8 GPUs)
  for (int r = 0; r < P.ranks; ++r) asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(P.arrive[r]) : "memory");
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(P.arrive[P.self]) : "memory");
    if (v >= P.ranks) break;
    if (global_timer_ns() - t0 > P.budget_ns) {  // a peer that never arrives: give up and say so
      if (P.status) atomicExch(P.status, kStatusExchangeWait);
      return;
    }
  }
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(P.arrive[P.self]), "r"(-P.ranks) : "memory");
}


// ---- the same exchange with the flag inside the data ---------------------------------------------------------------------
// Below a megabyte or so the exchange above is all latency: stores, a system-wide fence (one NVLink round trip), the
// count of finished CTAs, a second fence, the remote arrival, the poll: 12-14 us on two GPUs for a 57 KB slice. Here a
// 16-byte packet carries 8 bytes of y and the call's sequence number twice ({d0, seq, d1, seq}, the low-latency packet of
// collective libraries: an 8-byte half of a store arrives whole, so a half whose flag matches holds its data). Senders
// store packets straight into every peer's receive buffer, receivers poll the packets themselves and unpack them into
// y: no fence, no semaphore, one NVLink crossing on the critical path. Twice the bytes on the wire, so callers use it
// for small slices only.
//
// The sequence number lives in device memory (the call can sit in a replayed graph): every CTA reads it on entry, the
// last CTA to finish adds one. A peer can be one call ahead of a rank that still polls, never two, so every receive
// buffer has two halves and a call uses the half its sequence number's parity names: chosen on the device, the same on
// every rank, whatever the number of calls a replayed graph holds.
constexpr int kStatusExchangePoll = 7;  // a peer's packets did not arrive in time

struct PacketParams {
  uint8_t* y;                 // this rank's whole y
  uint4* box[kMaxRanks];      // every rank's receive buffer (peer-mapped): two halves of `ranks` regions; region r holds what rank r sent
  int64_t region;             // packets per region
  int64_t col0[kMaxRanks + 1];  // first column of every rank's slice; col0[ranks] = all columns
  uint32_t* seq;              // calls finished on this pair of buffers
  int* done;                  // CTAs finished (zero between calls)
  int ranks, self, M, elem;
  int64_t pitch;              // bytes between rows of y
  int* status;
  uint64_t budget_ns;
};

__global__ void __launch_bounds__(256) exchange_packets_kernel(const PacketParams P) {
  pdl_trigger();
  pdl_wait();  // the slice comes from the product before this kernel
  uint32_t seq;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seq) : "l"(P.seq) : "memory");
  const int64_t half = static_cast<int64_t>(seq & 1u) * P.ranks * P.region;  // this call's half of every receive buffer
  seq += 1;  // the flag of this call: never zero in a zeroed buffer's lifetime
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x, nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  {  // send: this rank's slice, 8 bytes per packet, to region `self` of every peer
    const int64_t per_row = (P.col0[P.self + 1] - P.col0[P.self]) * P.elem / 8, total = per_row * P.M;
    const uint8_t* src = P.y + P.col0[P.self] * P.elem;
    for (int64_t i = tid; i < total; i += nthreads) {
      const int64_t m = i / per_row;
      const uint2 d = *reinterpret_cast<const uint2*>(src + m * P.pitch + (i - m * per_row) * 8);
      for (int r = 0; r < P.ranks; ++r)
        if (r != P.self)
          asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(P.box[r] + half + P.self * P.region + i), "r"(d.x), "r"(seq), "r"(d.y), "r"(seq)
                       : "memory");
    }
  }
  const uint64_t t0 = global_timer_ns();
  bool gave_up = false;
  for (int r = 0; r < P.ranks && !gave_up; ++r) {  // receive: poll every peer's packets and put them where they belong in y
    if (r == P.self) continue;
    const int64_t per_row = (P.col0[r + 1] - P.col0[r]) * P.elem / 8, total = per_row * P.M;
    uint8_t* dst = P.y + P.col0[r] * P.elem;
    const uint4* in = P.box[P.self] + half + r * P.region;
    for (int64_t i = tid; i < total && !gave_up; i += nthreads) {
      uint32_t a, fa, b, fb;
      for (int spin = 0;; ++spin) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb) : "l"(in + i) : "memory");
        if (fa == seq && fb == seq) break;
        if ((spin & 63) == 63 && global_timer_ns() - t0 > P.budget_ns) {  // a peer that never sends: give up and say so
          gave_up = true;
          break;
        }
      }
      if (gave_up) break;
      const int64_t m = i / per_row;
      *reinterpret_cast<uint2*>(dst + m * P.pitch + (i - m * per_row) * 8) = make_uint2(a, b);
    }
  }
  if (gave_up && P.status) atomicExch(P.status, kStatusExchangePoll);
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence();
  int before;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(P.done) : "memory");
  if (before != static_cast<int>(gridDim.x) - 1) return;
  asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(P.done), "r"(0) : "memory");
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(P.seq), "r"(seq) : "memory");  // also after a timeout: the next call uses the next number
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int lx_b200_exchange_slices(void* const* y_all, int* const* arrivals, int ranks, int rank, int64_t col0, int cols,
                                       lx_dtype y_dtype, int ld_y, int M, void* stream) {
  if (!y_all || !arrivals || ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks) return kInvalid;
  if (M <= 0 || cols <= 0) return kOk;
  if (col0 < 0 || col0 + cols > ld_y || !valid_dtype(y_dtype)) return kInvalid;
  const int64_t elem = y_dtype == LX_BF16 ? 2 : 4;
  ExchangeParams P{};
  for (int r = 0; r < ranks; ++r) {
    if (!y_all[r] || !arrivals[r]) return kInvalid;
    P.y[r] = static_cast<uint8_t*>(y_all[r]) + col0 * elem;
    P.arrive[r] = arrivals[r];
  }
  P.done_local = arrivals[rank] + 1;
  P.ranks = ranks, P.self = rank, P.M = M;
  P.row_bytes = cols * elem;
  P.pitch = static_cast<int64_t>(ld_y) * elem;
  P.status = status_word();
  uint64_t ms = 1000;  // LX_B200_WAIT_MS: how long the wait for the peers may last (default 1000; read on every call)
  if (const char* v = std::getenv("LX_B200_WAIT_MS")) ms = static_cast<uint64_t>(std::max(1, std::min(10000, atoi(v))));
  P.budget_ns = ms * 1000000ull;
  bool v16 = P.row_bytes % 16 == 0 && P.pitch % 16 == 0;
  for (int r = 0; r < ranks; ++r) v16 = v16 && aligned(P.y[r], 16);
  const int V = v16 ? 16 : static_cast<int>(elem);
  const int64_t units = P.row_bytes / V * M * std::max(1, ranks - 1);
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(4 * 148, (units + 511) / 512)));
  auto s = static_cast<cudaStream_t>(stream);
  if (V == 16) return launch_kernel(exchange_kernel<16>, dim3(grid), dim3(256), 0, s, P);
  if (V == 4) return launch_kernel(exchange_kernel<4>, dim3(grid), dim3(256), 0, s, P);
  return launch_kernel(exchange_kernel<2>, dim3(grid), dim3(256), 0, s, P);
}

// bounds: ranks + 1 column indices, rank r owns columns [bounds[r], bounds[r + 1]) of the [M, ld_y] output. boxes: every
// rank's receive buffer of 2 * ranks * region packets of 16 bytes, zeroed once when allocated. seq and done: two zeroed
// words of this rank's own memory that belong to these boxes. Every slice row must be whole 8-byte pieces.
extern "C" int lx_b200_exchange_packets(void* y, void* const* boxes, int64_t region, uint32_t* seq, int* done, int ranks, int rank,
                                        const int64_t* bounds, lx_dtype y_dtype, int ld_y, int M, void* stream) {
  if (!y || !boxes || !seq || !done || !bounds || ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks) return kInvalid;
  if (M <= 0) return kOk;
  if (!valid_dtype(y_dtype) || region <= 0) return kInvalid;
  PacketParams P{};
  P.elem = y_dtype == LX_BF16 ? 2 : 4;
  P.pitch = static_cast<int64_t>(ld_y) * P.elem;
  if (!aligned(y, 8) || P.pitch % 8 != 0) return kNotSupported;
  int64_t most = 0;
  for (int r = 0; r <= ranks; ++r) {
    P.col0[r] = bounds[r];
    if (r > 0) {
      const int64_t cols = bounds[r] - bounds[r - 1];
      if (cols < 0 || (cols * P.elem) % 8 != 0 || (bounds[r - 1] * P.elem) % 8 != 0) return cols < 0 ? kInvalid : kNotSupported;
      if (cols * P.elem / 8 * M > region) return kInvalid;
      most = std::max(most, cols * P.elem / 8 * M);
    }
  }
  if (bounds[0] < 0 || bounds[ranks] > ld_y) return kInvalid;
  for (int r = 0; r < ranks; ++r) {
    if (!boxes[r] || !aligned(boxes[r], 16)) return kInvalid;
    P.box[r] = static_cast<uint4*>(boxes[r]);
  }
  P.y = static_cast<uint8_t*>(y);
  P.region = region;
  P.seq = seq, P.done = done;
  P.ranks = ranks, P.self = rank, P.M = M;
  P.status = status_word();
  uint64_t ms = 1000;  // LX_B200_WAIT_MS: how long the polls may last (default 1000; read on every call)
  if (const char* v = std::getenv("LX_B200_WAIT_MS")) ms = static_cast<uint64_t>(std::max(1, std::min(10000, atoi(v))));
  P.budget_ns = ms * 1000000ull;
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(148, (most + 255) / 256)));
  return launch_kernel(exchange_packets_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), P);
}
