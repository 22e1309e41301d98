// 2-D context parallelism behind the C ABI: a communicator over NCCL and the two
// triangle ops on one rank's tile of the pair tensor.
//
// Reference: the 2-D layer of FoldJAX - context_parallel, src/foldjax/models/_cp.py:259;
// _cannon_contract, src/foldjax/models/boltz2/models/triangle/triangle.py:132-212;
// ring_triangle_attention_2d, src/foldjax/models/_cp_attention.py:197-403. The reference
// runs inside shard_map on a square device grid and moves tiles with skews and ring hops;
// here the grid is R x C with C = m * R (1x2, 2x2, 2x4 on one 8-GPU box) and every tile
// travels straight between its owner and the rank that needs it: NVSwitch gives every pair of
// GPUs the same bandwidth, so a direct transfer replaces skew + hops. With one process per GPU
// the copy engines write the tiles into the receivers' CUDA-IPC-mapped workspaces (or the
// receivers read them) and NCCL only carries 4-byte tokens; otherwise the tiles are grouped
// ncclSend/ncclRecv (post_exchange below).
//
// Everything is enqueue-only. The exchange runs on the communicator's own stream and is
// fenced against the caller's stream with events in both directions, so the host never
// waits; remote tiles always land in this GPU's memory before a kernel reads them (no
// kernel is ever handed a peer pointer, and no TMA multicast exists anywhere).
//
// NCCL is reached through dlopen("libnccl.so.2") at the first communicator call: the
// library itself has no link-time dependency on it and still loads where NCCL is absent.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>
#include <algorithm>
#include <vector>

#include "host.cuh"

struct b200tri_comm {
  ncclComm_t nccl = nullptr;
  int world = 0, rank = 0, rows = 0, cols = 0, m = 0, r = 0, c = 0, device = 0;
  cudaStream_t stream = nullptr;  // exchange stream
  cudaEvent_t ev_ready = nullptr, ev_first = nullptr, ev_rest = nullptr;
  std::vector<cudaEvent_t> ev_part;  // fences of the groups of one exchange but the last: max(3, world) of them
  // Exchange workspace owned by the communicator (b200tri_comm_workspace) and, one process
  // per GPU, the peers' workspaces mapped into this process through CUDA IPC: tiles are then
  // pulled with device-to-device copies on the copy engines instead of NCCL's send/receive
  // kernels, and NCCL only carries the "tile ready" / "tile consumed" tokens.
  void* ws = nullptr;
  size_t ws_bytes = 0;
  std::vector<void*> peer_ws;  // [world], nullptr where not mapped (own rank, or no IPC)
  uint8_t* tokens = nullptr;   // device: 64-byte send slot + world x 64-byte receive slots
  bool one_process = false;    // created by b200tri_comm_init_all
  // Copies through the mapped workspaces: written into the receiver's workspace by the sender's
  // copy engines (push, the default: posted writes run at NVLink rate) or read out of the
  // sender's (pull), spread over `n_copy` streams so that several copy engines work at once.
  bool push = true;
  int n_copy = 1;
  int sm_reserve = 4;  // SMs left free beside a kernel that runs while tokens travel
  // Dry run (b200tri_cp_dry_run): no CUDA or NCCL call is made; the copies this rank would issue
  // and the launches it would make are written to this log instead, for checks on a CPU.
  std::vector<b200tri_cp_event>* dry = nullptr;
  int dry_group = 0;
  cudaStream_t copy_stream[4] = {nullptr, nullptr, nullptr, nullptr};  // [0] is `stream`
  cudaEvent_t ev_fork = nullptr, ev_join[4] = {nullptr, nullptr, nullptr, nullptr};
};

namespace b200 {
namespace {

// ------------------------------------------------------------------ NCCL entry points
struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

const Nccl* nccl_api() {
  static Nccl api;
  static bool tried = false;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return nullptr;
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(h, name);
    ok = ok && p != nullptr;
    return p;
  };
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
  api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
  api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
  api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
  api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
  api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  if (!ok) return nullptr;
  api.handle = h;
  return &api;
}

#define B200_NCCL_OK(api, expr)                                                                         \
  do {                                                                                                  \
    ncclResult_t _r = (expr);                                                                           \
    if (_r != ncclSuccess) {                                                                            \
      b200::set_error("%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), __FILE__, __LINE__);   \
      return B200TRI_ERR_CUDA;                                                                          \
    }                                                                                                   \
  } while (0)

// ------------------------------------------------------------------------------ the plan
// One message of an exchange: `what` names the sender's local array, `block` the row block
// of it that travels (-1 = the whole tile), slot0/slot1 the position in the receiver's panel.
enum { WHAT_A = 0, WHAT_B = 1, WHAT_KV = 2, WHAT_BIAS = 3 };
using Msg = b200tri_cp_msg;

struct Grid {
  int rows, cols, m;
  int rank(int r, int c) const { return r * cols + c; }
};

// The global message list of an op: the same on every rank, so that the sends of one rank
// and the receives of its peer are posted in the same relative order.
std::vector<Msg> build_plan(const Grid& g, int op) {
  std::vector<Msg> msgs;
  for (int dst = 0; dst < g.rows * g.cols; ++dst) {
    const int r = dst / g.cols, c = dst % g.cols;
    switch (op) {
      case B200TRI_CP_TRIMUL_OUTGOING:
        // out[I_r, J_c] = sum_c' a[I_r, K_c'] . b[J_c, K_c']^T: a tile of the row peer (r, c'),
        // and the row block of b whose rows are J_c, which lives on (c / m, c').
        for (int cp = 0; cp < g.cols; ++cp) {
          msgs.push_back({g.rank(r, cp), dst, WHAT_A, -1, cp, 0});
          msgs.push_back({g.rank(c / g.m, cp), dst, WHAT_B, c % g.m, cp, 0});
        }
        break;
      case B200TRI_CP_TRIMUL_INCOMING:
        // out[I_r, J_c] = sum_r'' a[K_r'', I_r]^T . b[K_r'', J_c], projected through swapped
        // strides: output row block s needs a' of (r'', r * m + s); all need b' of (r'', c).
        for (int rp = 0; rp < g.rows; ++rp) {
          for (int s = 0; s < g.m; ++s) msgs.push_back({g.rank(rp, r * g.m + s), dst, WHAT_A, -1, s, rp});
          msgs.push_back({g.rank(rp, c), dst, WHAT_B, -1, rp, 0});
        }
        break;
      case B200TRI_CP_TRIATT_STARTING:
        // rows I_r, queries J_c, keys of every K_c': K/V of (r, c'); the bias of (J_c, K_c') is
        // row block c % m of the bias of (c / m, c').
        for (int cp = 0; cp < g.cols; ++cp) {
          msgs.push_back({g.rank(r, cp), dst, WHAT_KV, -1, cp, 0});
          msgs.push_back({g.rank(c / g.m, cp), dst, WHAT_BIAS, c % g.m, cp, 0});
        }
        break;
      case B200TRI_CP_TRIATT_ENDING:
        // transposed frame: rows J_c, queries I_r, keys of every I_r'': K/V of (r'', c); the
        // bias of (J_{r*m+s}, I_r'') is the whole bias of (r'', r * m + s).
        for (int rp = 0; rp < g.rows; ++rp) {
          msgs.push_back({g.rank(rp, c), dst, WHAT_KV, -1, rp, 0});
          for (int s = 0; s < g.m; ++s) msgs.push_back({g.rank(rp, r * g.m + s), dst, WHAT_BIAS, -1, rp, s});
        }
        break;
      default:
        break;
    }
  }
  return msgs;
}

struct Piece {
  size_t off;  // byte offset inside the workspace (of the rank whose array it is)
  size_t bytes;
};

// Byte offsets of 1 KiB-aligned pieces of a workspace.
struct Offsets {
  size_t off = 0;
  size_t take(size_t bytes) {
    off = (off + 1023) / 1024 * 1024;
    const size_t r = off;
    off += bytes;
    return r;
  }
  size_t total() const { return (off + 1023) / 1024 * 1024; }
};

// Round of every message of an exchange (-1: not wanted, or local). In one round every rank
// sends at most one tile and receives at most one, and there are no more rounds than the busiest
// rank has messages: an edge colouring of the bipartite sender/receiver graph (alternating-path
// recolouring), identical on every rank. Copies issued in this order keep every link busy
// without several senders serving the same receiver at the same time. `big` messages are coloured
// first, so they share the early rounds.
template <typename Want, typename Big>
std::vector<int> copy_rounds(const std::vector<Msg>& msgs, int world, Want want, Big big) {
  std::vector<int> round(msgs.size(), -1), edges;
  std::vector<int> deg(2 * static_cast<size_t>(world), 0);
  for (int pass = 0; pass < 2; ++pass)
    for (size_t i = 0; i < msgs.size(); ++i)
      if (want(msgs[i]) && msgs[i].src != msgs[i].dst && big(msgs[i]) == (pass == 0)) {
        edges.push_back(static_cast<int>(i));
        ++deg[msgs[i].src];
        ++deg[world + msgs[i].dst];
      }
  const int colours = edges.empty() ? 0 : *std::max_element(deg.begin(), deg.end());
  // at[node][colour] = message holding that colour at the node (senders 0..world, receivers after)
  std::vector<std::vector<int>> at(2 * static_cast<size_t>(world), std::vector<int>(colours, -1));
  auto free_at = [&](int node) {
    int c = 0;
    while (at[node][c] >= 0) ++c;  // a node has at most `colours` messages, this one not yet placed
    return c;
  };
  for (int e : edges) {
    const int u = msgs[e].src, v = world + msgs[e].dst;
    const int a = free_at(u), b = free_at(v);
    if (at[v][a] >= 0) {  // a is taken at the receiver: swap a and b along the path that starts there
      std::vector<int> path;
      for (int node = v, c = a; at[node][c] >= 0; c = c == a ? b : a) {
        const int f = at[node][c];
        path.push_back(f);
        node = node >= world ? msgs[f].src : world + msgs[f].dst;
      }
      for (int f : path) at[msgs[f].src][round[f]] = at[world + msgs[f].dst][round[f]] = -1;
      for (int f : path) {
        round[f] = round[f] == a ? b : a;
        at[msgs[f].src][round[f]] = at[world + msgs[f].dst][round[f]] = f;
      }
    }
    round[e] = a;
    at[u][a] = at[v][a] = e;
  }
  return round;
}

// Post this rank's share of `msgs` (those accepted by `want`). `views(msg, send, who, out)`
// lists the pieces of a message as offsets into the workspace: on the send side inside the
// workspace of rank `who` = msg.src, on the receive side inside this rank's. Local messages
// are device copies on the caller's stream. Remote ones travel
//  * as one NCCL group of sends and receives on the exchange stream, or
//  * when every peer's workspace is mapped here (`pull`): the receiver copies each piece out
//    of the sender's workspace with a device-to-device copy (copy engines, full NVLink rate);
//    NCCL carries a 4-byte "ready" token from sender to receiver before the copies and a
//    "consumed" token back after them, so a sender never overwrites a tile that is being read.
template <typename Want, typename Views>
int post_exchange(b200tri_comm* cm, uint8_t* ws, bool pull, const std::vector<Msg>& msgs, Want want, Views views,
                  cudaStream_t compute, int wide_what = -1) {
  auto big = [&](const Msg& msg) { return msg.what == wide_what; };  // messages larger than the others
  std::vector<Piece> send, recv;
  auto remote = [&](const Msg& msg) {
    return want(msg) && msg.src != msg.dst && (msg.src == cm->rank || msg.dst == cm->rank);
  };
  if (cm->dry) {
    // the copies this rank would issue, in issue order: local ones, then the remote ones it
    // sends (push) or fetches (pull) round by round
    const int group = cm->dry_group++;
    const std::vector<int> round = copy_rounds(msgs, cm->world, want, big);
    int n_rounds = 0;
    for (int r : round) n_rounds = std::max(n_rounds, r + 1);
    auto log = [&](const Msg& msg, int kind, int rnd) {
      send.clear();
      recv.clear();
      views(msg, true, msg.src, send);
      views(msg, false, msg.dst, recv);
      for (size_t i = 0; i < send.size(); ++i) {
        b200tri_cp_event e = {};
        e.kind = kind;
        e.group = group;
        e.round = rnd;
        e.src = msg.src;
        e.dst = msg.dst;
        e.what = msg.what;
        e.block = msg.block;
        e.slot0 = msg.slot0;
        e.slot1 = msg.slot1;
        e.src_off = static_cast<int64_t>(send[i].off);
        e.dst_off = static_cast<int64_t>(recv[i].off);
        e.bytes = static_cast<int64_t>(send[i].bytes);
        cm->dry->push_back(e);
      }
    };
    for (const Msg& msg : msgs)
      if (want(msg) && msg.src == cm->rank && msg.dst == cm->rank) log(msg, B200TRI_CP_EVENT_LOCAL_COPY, -1);
    for (int r = 0; r < n_rounds; ++r)
      for (size_t i = 0; i < msgs.size(); ++i)
        if (round[i] == r && (pull ? (cm->push ? msgs[i].src : msgs[i].dst) : msgs[i].src) == cm->rank)
          log(msgs[i], B200TRI_CP_EVENT_COPY, r);
    return B200TRI_OK;
  }
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  // with timing on, the span of this exchange on the exchange stream (it starts when the stream
  // has seen the caller's "tiles are ready" event, so it is transfer time plus peer skew)
  TimedLaunch timed(K_CP_EXCHANGE, cm->stream);
  // local messages
  for (const Msg& msg : msgs) {
    if (!want(msg) || msg.src != cm->rank || msg.dst != cm->rank) continue;
    send.clear();
    recv.clear();
    views(msg, true, cm->rank, send);
    views(msg, false, cm->rank, recv);
    for (size_t i = 0; i < send.size(); ++i)
      if (send[i].off != recv[i].off)
        B200_CUDA_OK(cudaMemcpyAsync(ws + recv[i].off, ws + send[i].off, send[i].bytes, cudaMemcpyDeviceToDevice, compute));
  }
  bool any = false;
  for (const Msg& msg : msgs) any = any || remote(msg);
  if (!any) return B200TRI_OK;
  if (!pull) {
    B200_NCCL_OK(api, api->GroupStart());
    for (const Msg& msg : msgs) {
      if (!remote(msg)) continue;
      send.clear();
      recv.clear();
      if (msg.src == cm->rank) views(msg, true, cm->rank, send);
      if (msg.dst == cm->rank) views(msg, false, cm->rank, recv);
      for (const Piece& p : send) B200_NCCL_OK(api, api->Send(ws + p.off, p.bytes, ncclUint8, msg.dst, cm->nccl, cm->stream));
      for (const Piece& p : recv) B200_NCCL_OK(api, api->Recv(ws + p.off, p.bytes, ncclUint8, msg.src, cm->nccl, cm->stream));
    }
    B200_NCCL_OK(api, api->GroupEnd());
    return B200TRI_OK;
  }
  // tokens: slot 0 is what this rank sends, slot 1 + peer what it receives from that peer.
  // to_receiver = true: one token per message from its sender to its receiver; false: the reverse.
  auto token_round = [&](bool to_receiver) -> int {
    B200_NCCL_OK(api, api->GroupStart());
    for (const Msg& msg : msgs) {
      if (!remote(msg)) continue;
      const bool i_send = to_receiver ? msg.src == cm->rank : msg.dst == cm->rank;
      const int peer = msg.src == cm->rank ? msg.dst : msg.src;
      if (i_send)
        B200_NCCL_OK(api, api->Send(cm->tokens, 4, ncclUint8, peer, cm->nccl, cm->stream));
      else
        B200_NCCL_OK(api, api->Recv(cm->tokens + 64 * (1 + peer), 4, ncclUint8, peer, cm->nccl, cm->stream));
    }
    B200_NCCL_OK(api, api->GroupEnd());
    return B200TRI_OK;
  };
  const bool push = cm->push;
  int rc;
  {
    // with timing on: how long the peers were waited for
    TimedLaunch waited(K_CP_READY, cm->stream);
    // pull: every sender's tiles are complete. push: every receiver has reached this exchange,
    // so nothing of its earlier work still reads the slots about to be written.
    rc = token_round(!push);
  }
  if (rc) return rc;
  TimedLaunch copied(K_CP_COPY, cm->stream);  // ... and the copies themselves (plus the closing round)
  if (cm->n_copy > 1) {
    B200_CUDA_OK(cudaEventRecord(cm->ev_fork, cm->stream));
    for (int i = 1; i < cm->n_copy; ++i) B200_CUDA_OK(cudaStreamWaitEvent(cm->copy_stream[i], cm->ev_fork, 0));
  }
  // Order of the copies: rounds in which every rank sends at most one tile and receives at most
  // one (a greedy edge colouring of the whole exchange, the same on every rank, busiest ranks
  // first). Taken in plan order instead, several senders serve the same receiver at the same
  // time while other receivers wait, and the exchange runs at half the link rate.
  std::vector<int> order;  // indices into msgs of the copies this rank issues, round by round
  {
    const std::vector<int> round = copy_rounds(msgs, cm->world, want, big);
    int n_rounds = 0;
    for (int r : round) n_rounds = std::max(n_rounds, r + 1);
    for (int r = 0; r < n_rounds; ++r)
      for (size_t i = 0; i < msgs.size(); ++i)
        if (round[i] == r && (push ? msgs[i].src : msgs[i].dst) == cm->rank) order.push_back(static_cast<int>(i));
  }
  for (int idx : order) {
    const Msg& msg = msgs[idx];
    send.clear();
    recv.clear();
    views(msg, true, msg.src, send);
    views(msg, false, msg.dst, recv);
    const int peer = push ? msg.dst : msg.src;
    uint8_t* theirs = static_cast<uint8_t*>(cm->peer_ws[peer]);
    for (size_t i = 0; i < send.size(); ++i) {
      const uint8_t* from = push ? ws + send[i].off : theirs + send[i].off;
      uint8_t* to = push ? theirs + recv[i].off : ws + recv[i].off;
      // every piece is cut into n_copy parts, one per stream: two copy engines working on one
      // tile come closer to the link rate than one
      const size_t part = (send[i].bytes / cm->n_copy + 1023) / 1024 * 1024;
      for (int k = 0; k < cm->n_copy; ++k) {
        const size_t lo = std::min(send[i].bytes, part * k), hi = std::min(send[i].bytes, part * (k + 1));
        if (hi > lo)
          B200_CUDA_OK(cudaMemcpyAsync(to + lo, from + lo, hi - lo, cudaMemcpyDeviceToDevice, cm->copy_stream[k]));
      }
    }
  }
  for (int i = 1; i < cm->n_copy; ++i) {
    B200_CUDA_OK(cudaEventRecord(cm->ev_join[i], cm->copy_stream[i]));
    B200_CUDA_OK(cudaStreamWaitEvent(cm->stream, cm->ev_join[i], 0));
  }
  // pull: every tile has been read, the senders may reuse their buffers. push: every tile has
  // been written (the sender's own buffers are protected by its stream order).
  return token_round(push);
}

// CUDA calls of the ops that a dry run skips
#define CP_CUDA(cm, call)               \
  do {                                  \
    if (!(cm)->dry) B200_CUDA_OK(call); \
  } while (0)

// a launch the op would make, for the dry-run log: offsets are relative to the workspace
// (off[0..2]) and to the rank's tile (off[3])
void log_launch(b200tri_comm* cm, int kind, int group, int n_i, int n_j, int64_t o0, int64_t o1, int64_t o2, int64_t o3) {
  if (!cm->dry) return;
  b200tri_cp_event e = {};
  e.kind = kind;
  e.group = group;
  e.round = -1;
  e.src = e.dst = cm->rank;
  e.what = e.block = e.slot0 = e.slot1 = -1;
  e.n_i = n_i;
  e.n_j = n_j;
  e.off[0] = o0;
  e.off[1] = o1;
  e.off[2] = o2;
  e.off[3] = o3;
  cm->dry->push_back(e);
}

int check_comm(const b200tri_comm* cm, const char* who) {
  if (cm != nullptr && cm->dry != nullptr) return B200TRI_OK;
  B200_REQUIRE(cm != nullptr && cm->nccl != nullptr, B200TRI_ERR_INVALID, "%s: null or destroyed communicator", who);
  int dev = -1;
  B200_CUDA_OK(cudaGetDevice(&dev));
  B200_REQUIRE(dev == cm->device, B200TRI_ERR_INVALID, "%s: the communicator belongs to device %d, current device is %d",
               who, cm->device, dev);
  return B200TRI_OK;
}

int finish_init(b200tri_comm* cm, int world, int rank, int rows, int cols) {
  cm->world = world;
  cm->rank = rank;
  cm->rows = rows;
  cm->cols = cols;
  cm->m = cols / rows;
  cm->r = rank / cols;
  cm->c = rank % cols;
  B200_CUDA_OK(cudaGetDevice(&cm->device));
  B200_CUDA_OK(cudaStreamCreateWithFlags(&cm->stream, cudaStreamNonBlocking));
  B200_CUDA_OK(cudaEventCreateWithFlags(&cm->ev_ready, cudaEventDisableTiming));
  B200_CUDA_OK(cudaEventCreateWithFlags(&cm->ev_first, cudaEventDisableTiming));
  B200_CUDA_OK(cudaEventCreateWithFlags(&cm->ev_rest, cudaEventDisableTiming));
  cm->ev_part.assign(world > 3 ? world : 3, nullptr);
  for (cudaEvent_t& e : cm->ev_part) B200_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  B200_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&cm->tokens), 64 * (1 + static_cast<size_t>(world))));
  B200_CUDA_OK(cudaMemset(cm->tokens, 0, 64 * (1 + static_cast<size_t>(world))));
  cm->copy_stream[0] = cm->stream;
  B200_CUDA_OK(cudaEventCreateWithFlags(&cm->ev_fork, cudaEventDisableTiming));
  for (int i = 1; i < 4; ++i) {
    B200_CUDA_OK(cudaStreamCreateWithFlags(&cm->copy_stream[i], cudaStreamNonBlocking));
    B200_CUDA_OK(cudaEventCreateWithFlags(&cm->ev_join[i], cudaEventDisableTiming));
  }
  return B200TRI_OK;
}

// Every rank contributes 64 bytes (`mine`) and receives every rank's into all[world][64]:
// an all-gather over the communicator's send/receive path. Host-synchronous (set-up only).
int gather_64(b200tri_comm* cm, const void* mine, uint8_t* all) {
  const Nccl* api = nccl_api();
  B200_CUDA_OK(cudaMemcpyAsync(cm->tokens, mine, 64, cudaMemcpyHostToDevice, cm->stream));
  B200_NCCL_OK(api, api->GroupStart());
  for (int peer = 0; peer < cm->world; ++peer) {
    if (peer == cm->rank) continue;
    B200_NCCL_OK(api, api->Send(cm->tokens, 64, ncclUint8, peer, cm->nccl, cm->stream));
    B200_NCCL_OK(api, api->Recv(cm->tokens + 64 * (1 + peer), 64, ncclUint8, peer, cm->nccl, cm->stream));
  }
  B200_NCCL_OK(api, api->GroupEnd());
  B200_CUDA_OK(cudaMemcpyAsync(all, cm->tokens + 64, 64 * static_cast<size_t>(cm->world), cudaMemcpyDeviceToHost, cm->stream));
  B200_CUDA_OK(cudaStreamSynchronize(cm->stream));
  memcpy(all + 64 * static_cast<size_t>(cm->rank), mine, 64);
  return B200TRI_OK;
}

void unmap_peers(b200tri_comm* cm) {
  for (void* p : cm->peer_ws)
    if (p) cudaIpcCloseMemHandle(p);
  cm->peer_ws.clear();
}

int check_grid(int world, int rows, int cols) {
  B200_REQUIRE(rows >= 1 && cols >= 1 && rows * cols == world, B200TRI_ERR_INVALID,
               "context-parallel grid %dx%d does not use %d ranks", rows, cols, world);
  B200_REQUIRE(cols % rows == 0, B200TRI_ERR_UNSUPPORTED,
               "unsupported context-parallel grid %dx%d: columns must be a multiple of rows", rows, cols);
  return B200TRI_OK;
}

struct TileDims {
  int n, n_r, n_c;
};

int tile_dims(const b200tri_comm* cm, int n, TileDims* d) {
  B200_REQUIRE(n > 0 && n % cm->cols == 0, B200TRI_ERR_INVALID,
               "token count %d is not divisible by the %d grid columns; pad it first", n, cm->cols);
  d->n = n;
  d->n_r = n / cm->rows;
  d->n_c = n / cm->cols;
  return B200TRI_OK;
}

// ---------------------------------------------------------------- tri-mult workspace
struct TrimulPlan {
  int n_outer, n_inner, n_src, n_k, ld, ldt, rpb, t_rpb;
  size_t blk;  // elements of one n_c-row block of channel-major data [128][n_c][ld]
  size_t a_all, a_loc, b_all, b_loc, t, proj, fin, total;  // byte offsets
};

TrimulPlan trimul_plan(const b200tri_comm* cm, const TileDims& d, bool incoming) {
  TrimulPlan p;
  const int R = cm->rows, C = cm->cols, m = cm->m;
  p.n_outer = incoming ? d.n_c : d.n_r;
  p.n_inner = incoming ? d.n_r : d.n_c;
  p.n_src = incoming ? R : C;
  p.n_k = p.n_inner;
  p.ld = round_up(p.n_inner, 64);
  p.ldt = round_up(d.n_c, 64);
  p.rpb = d.n_c % 64 == 0 ? 64 : d.n_c;
  p.t_rpb = p.rpb == 64 ? 64 : d.n_r;
  p.blk = static_cast<size_t>(128) * d.n_c * p.ld;
  Offsets w;
  auto off = [&](size_t elems, size_t esize) { return w.take(elems * esize); };
  if (!incoming) {
    p.a_all = off(static_cast<size_t>(C) * m * p.blk, 2);  // slot c' <- a of (r, c')
    p.b_loc = off(static_cast<size_t>(m) * p.blk, 2);
    p.b_all = off(static_cast<size_t>(C) * p.blk, 2);      // slot c' <- block c % m of b of (c / m, c')
    p.a_loc = p.a_all + static_cast<size_t>(cm->c) * m * p.blk * 2;
  } else {
    p.a_all = off(static_cast<size_t>(m) * R * p.blk, 2);  // slot (s, r'') <- a' of (r'', r * m + s)
    p.a_loc = off(p.blk, 2);
    p.b_all = off(static_cast<size_t>(R) * p.blk, 2);      // slot r'' <- b' of (r'', c)
    p.b_loc = p.b_all + static_cast<size_t>(cm->r) * p.blk * 2;
  }
  p.t = off(static_cast<size_t>(128) * d.n_r * p.ldt, 2);
  p.proj = off(b200tri_trimul_project_workspace_bytes(), 1);
  p.fin = off(b200tri_trimul_finish_workspace_bytes(), 1);
  p.total = w.total();
  return p;
}

// ---------------------------------------------------------------- tri-attn workspace
struct TriattPlan {
  int n_outer, n_inner, n_q, tiles, own, ld;
  size_t q, k_all, vt_all, bias_loc, bias_all, o, acc, rmax, rsum, proj, core, fin, total;
  size_t k_tile, vt_tile, bias_tile;  // bytes of one key tile's K, V^T and bias
};

TriattPlan triatt_plan(const b200tri_comm* cm, const TileDims& d, bool starting) {
  TriattPlan p;
  p.n_outer = starting ? d.n_r : d.n_c;
  p.n_inner = starting ? d.n_c : d.n_r;
  p.n_q = p.n_inner;
  p.tiles = starting ? cm->cols : cm->rows;
  p.own = starting ? cm->c : cm->r;
  p.ld = round_up(p.n_inner, 64);
  p.k_tile = static_cast<size_t>(p.n_outer) * p.n_inner * 128 * 2;
  p.vt_tile = static_cast<size_t>(p.n_outer) * 128 * p.ld * 2;
  p.bias_tile = static_cast<size_t>(4) * p.n_q * p.ld * 2;
  Offsets w;
  auto off = [&](size_t bytes) { return w.take(bytes); };
  p.q = off(p.k_tile);
  p.k_all = off(p.k_tile * p.tiles);
  p.vt_all = off(p.vt_tile * p.tiles);
  p.bias_loc = off(static_cast<size_t>(4) * p.n_outer * p.ld * 2);
  p.bias_all = off(p.bias_tile * p.tiles);
  p.o = off(static_cast<size_t>(p.n_outer) * p.n_q * 128 * 2);
  p.acc = off(static_cast<size_t>(p.n_outer) * p.n_q * 128 * 4);
  p.rmax = off(static_cast<size_t>(p.n_outer) * 4 * p.n_q * 4);
  p.rsum = off(static_cast<size_t>(p.n_outer) * 4 * p.n_q * 4);
  p.proj = off(b200tri_triatt_project_workspace_bytes());
  p.core = off(b200tri_triatt_core_multi_workspace_bytes(p.n_outer, p.n_inner, p.tiles));
  p.fin = off(b200tri_triatt_finish_workspace_bytes());
  p.total = w.total();
  return p;
}

}  // namespace
}  // namespace b200

using namespace b200;

// ============================================================================ C ABI
extern "C" int b200tri_cp_plan(int32_t rows, int32_t cols, int32_t op, b200tri_cp_msg* out, int32_t capacity) {
  if (check_grid(rows * cols, rows, cols)) return -1;
  if (op < B200TRI_CP_TRIMUL_OUTGOING || op > B200TRI_CP_TRIATT_ENDING) {
    set_error("cp_plan: unknown op %d", op);
    return -1;
  }
  const std::vector<Msg> msgs = build_plan(Grid{rows, cols, cols / rows}, op);
  if (out)
    for (size_t i = 0; i < msgs.size() && static_cast<int32_t>(i) < capacity; ++i) out[i] = msgs[i];
  return static_cast<int>(msgs.size());
}

extern "C" int b200tri_cp_rounds(int32_t rows, int32_t cols, int32_t op, int32_t what, int32_t* round, int32_t capacity) {
  if (check_grid(rows * cols, rows, cols)) return -1;
  if (op < B200TRI_CP_TRIMUL_OUTGOING || op > B200TRI_CP_TRIATT_ENDING) {
    set_error("cp_rounds: unknown op %d", op);
    return -1;
  }
  const std::vector<Msg> msgs = build_plan(Grid{rows, cols, cols / rows}, op);
  // the tile of an outgoing tri-mult `a` message spans cols / rows blocks, every other message one
  const bool wide = op == B200TRI_CP_TRIMUL_OUTGOING && cols > rows;
  const std::vector<int> r = copy_rounds(
      msgs, rows * cols, [&](const Msg& m) { return what < 0 || m.what == what; },
      [&](const Msg& m) { return wide && m.what == WHAT_A; });
  if (round)
    for (size_t i = 0; i < r.size() && static_cast<int32_t>(i) < capacity; ++i) round[i] = r[i];
  return static_cast<int>(r.size());
}

extern "C" int b200tri_comm_unique_id(void* id128) {
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  B200_REQUIRE(id128 != nullptr, B200TRI_ERR_INVALID, "comm_unique_id: null buffer");
  static_assert(sizeof(ncclUniqueId) == B200TRI_COMM_ID_BYTES, "NCCL unique id size");
  B200_NCCL_OK(api, api->GetUniqueId(static_cast<ncclUniqueId*>(id128)));
  return B200TRI_OK;
}

extern "C" int b200tri_comm_init(b200tri_comm** out, const void* id128, int32_t world, int32_t rank, int32_t rows,
                                 int32_t cols) {
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  B200_REQUIRE(out && id128, B200TRI_ERR_INVALID, "comm_init: null argument");
  B200_REQUIRE(rank >= 0 && rank < world, B200TRI_ERR_INVALID, "comm_init: rank %d outside [0, %d)", rank, world);
  int rc = check_grid(world, rows, cols);
  if (rc) return rc;
  b200tri_comm* cm = new b200tri_comm;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclResult_t r = api->CommInitRank(&cm->nccl, world, id, rank);
  if (r != ncclSuccess) {
    set_error("ncclCommInitRank failed: %s", api->GetErrorString(r));
    delete cm;
    return B200TRI_ERR_CUDA;
  }
  rc = finish_init(cm, world, rank, rows, cols);
  if (rc) {
    b200tri_comm_destroy(cm);
    return rc;
  }
  *out = cm;
  return B200TRI_OK;
}

extern "C" int b200tri_comm_init_all(b200tri_comm** out, const int32_t* devices, int32_t world, int32_t rows,
                                     int32_t cols) {
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  B200_REQUIRE(out && world >= 1 && world <= 64, B200TRI_ERR_INVALID, "comm_init_all: bad arguments");
  int rc = check_grid(world, rows, cols);
  if (rc) return rc;
  std::vector<ncclComm_t> comms(world);
  std::vector<int> devs(world);
  for (int i = 0; i < world; ++i) devs[i] = devices ? devices[i] : i;
  B200_NCCL_OK(api, api->CommInitAll(comms.data(), world, devs.data()));
  int prev = 0;
  B200_CUDA_OK(cudaGetDevice(&prev));
  for (int i = 0; i < world; ++i) {
    out[i] = new b200tri_comm;
    out[i]->nccl = comms[i];
    out[i]->one_process = true;
    B200_CUDA_OK(cudaSetDevice(devs[i]));
    rc = finish_init(out[i], world, i, rows, cols);
    if (rc) break;
  }
  cudaSetDevice(prev);
  return rc;
}

extern "C" int b200tri_comm_destroy(b200tri_comm* cm) {
  if (!cm) return B200TRI_OK;
  const Nccl* api = nccl_api();
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(cm->device);
  if (cm->stream) cudaStreamSynchronize(cm->stream);
  unmap_peers(cm);
  if (cm->ws) cudaFree(cm->ws);
  if (cm->tokens) cudaFree(cm->tokens);
  if (cm->nccl && api) api->CommDestroy(cm->nccl);
  if (cm->ev_ready) cudaEventDestroy(cm->ev_ready);
  if (cm->ev_first) cudaEventDestroy(cm->ev_first);
  if (cm->ev_rest) cudaEventDestroy(cm->ev_rest);
  for (cudaEvent_t e : cm->ev_part)
    if (e) cudaEventDestroy(e);
  if (cm->ev_fork) cudaEventDestroy(cm->ev_fork);
  for (int i = 1; i < 4; ++i) {
    if (cm->copy_stream[i]) cudaStreamSynchronize(cm->copy_stream[i]);
    if (cm->ev_join[i]) cudaEventDestroy(cm->ev_join[i]);
    if (cm->copy_stream[i]) cudaStreamDestroy(cm->copy_stream[i]);
  }
  if (cm->stream) cudaStreamDestroy(cm->stream);
  cudaSetDevice(prev);
  delete cm;
  return B200TRI_OK;
}

// The communicator's own exchange workspace: (re)allocated here - set-up time, never inside an
// op - and, with one process per GPU, mapped into every peer through CUDA IPC, so that the ops
// can pull tiles with device-to-device copies. Collective: every rank calls it with the same
// size at the same point. Host-synchronous.
extern "C" int b200tri_comm_workspace(b200tri_comm* cm, size_t bytes, void** out) {
  int rc = check_comm(cm, "comm_workspace");
  if (rc) return rc;
  B200_REQUIRE(out != nullptr && bytes > 0, B200TRI_ERR_INVALID, "comm_workspace: null result pointer or zero size");
  if (cm->ws && cm->ws_bytes >= bytes) {
    *out = cm->ws;
    return B200TRI_OK;
  }
  B200_CUDA_OK(cudaDeviceSynchronize());
  unmap_peers(cm);
  if (cm->ws) B200_CUDA_OK(cudaFree(cm->ws));
  cm->ws = nullptr;
  cm->ws_bytes = 0;
  B200_CUDA_OK(cudaMalloc(&cm->ws, bytes));
  cm->ws_bytes = bytes;
  *out = cm->ws;
  if (cm->one_process || cm->world == 1) return B200TRI_OK;  // tiles travel as NCCL sends / receives
  // exchange the IPC handles, map the peers, and agree on the outcome
  cudaIpcMemHandle_t mine;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  B200_CUDA_OK(cudaIpcGetMemHandle(&mine, cm->ws));
  std::vector<uint8_t> all(64 * static_cast<size_t>(cm->world));
  if ((rc = gather_64(cm, &mine, all.data()))) return rc;
  cm->peer_ws.assign(cm->world, nullptr);
  uint8_t ok[64] = {1};
  for (int peer = 0; peer < cm->world; ++peer) {
    if (peer == cm->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, all.data() + 64 * static_cast<size_t>(peer), 64);
    if (cudaIpcOpenMemHandle(&cm->peer_ws[peer], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      cm->peer_ws[peer] = nullptr;
      ok[0] = 0;
    }
  }
  if ((rc = gather_64(cm, ok, all.data()))) return rc;
  for (int peer = 0; peer < cm->world; ++peer)
    if (all[64 * static_cast<size_t>(peer)] == 0) ok[0] = 0;
  if (!ok[0]) unmap_peers(cm);  // some rank could not map a peer: every rank stays on sends / receives
  return B200TRI_OK;
}

// 1 if the ops called with workspace = NULL move their tiles through mapped peer memory.
extern "C" int b200tri_comm_pulls(const b200tri_comm* cm) { return cm && !cm->peer_ws.empty() ? 1 : 0; }

extern "C" int b200tri_comm_configure(b200tri_comm* cm, int32_t push, int32_t copy_streams, int32_t sm_reserve) {
  int rc = check_comm(cm, "comm_configure");
  if (rc) return rc;
  B200_REQUIRE(copy_streams >= 1 && copy_streams <= 4, B200TRI_ERR_INVALID,
               "comm_configure: 1 to 4 copy streams, got %d", copy_streams);
  B200_CUDA_OK(cudaStreamSynchronize(cm->stream));  // set-up time: nothing of an exchange is in flight
  B200_REQUIRE(sm_reserve >= 0 && sm_reserve <= 64, B200TRI_ERR_INVALID,
               "comm_configure: 0 to 64 reserved SMs, got %d", sm_reserve);
  cm->push = push != 0;
  cm->n_copy = copy_streams;
  cm->sm_reserve = sm_reserve;
  return B200TRI_OK;
}

extern "C" int b200tri_comm_info(const b200tri_comm* cm, int32_t* world, int32_t* rank, int32_t* rows, int32_t* cols) {
  B200_REQUIRE(cm != nullptr, B200TRI_ERR_INVALID, "comm_info: null communicator");
  if (world) *world = cm->world;
  if (rank) *rank = cm->rank;
  if (rows) *rows = cm->rows;
  if (cols) *cols = cm->cols;
  return B200TRI_OK;
}

extern "C" int b200tri_comm_group_start(void) {
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  B200_NCCL_OK(api, api->GroupStart());
  return B200TRI_OK;
}

extern "C" int b200tri_comm_group_end(void) {
  const Nccl* api = nccl_api();
  B200_REQUIRE(api != nullptr, B200TRI_ERR_CUDA, "libnccl.so.2 could not be loaded");
  B200_NCCL_OK(api, api->GroupEnd());
  return B200TRI_OK;
}

// Every rank sends `bytes` from `shard` to every other rank and receives theirs into
// gathered[src * bytes ...] (its own shard is copied): an all-gather through the very
// send/receive path the ops use. The host compares the result with what was sent.
extern "C" int b200tri_comm_probe(b200tri_comm* cm, const void* shard, void* gathered, size_t bytes,
                                  b200tri_stream_t stream_) {
  int rc = check_comm(cm, "comm_probe");
  if (rc) return rc;
  B200_REQUIRE(shard && gathered && bytes > 0, B200TRI_ERR_INVALID, "comm_probe: null buffer or zero size");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  std::vector<Msg> msgs;
  for (int dst = 0; dst < cm->world; ++dst)
    for (int src = 0; src < cm->world; ++src) msgs.push_back({src, dst, WHAT_A, -1, src, 0});
  B200_CUDA_OK(cudaEventRecord(cm->ev_ready, stream));
  B200_CUDA_OK(cudaStreamWaitEvent(cm->stream, cm->ev_ready, 0));
  // absolute addresses as "offsets" from a null base; always the NCCL path (the probe tests it)
  rc = post_exchange(
      cm, nullptr, false, msgs, [](const Msg&) { return true; },
      [&](const Msg& msg, bool send, int, std::vector<Piece>& out) {
        if (send)
          out.push_back({reinterpret_cast<size_t>(shard), bytes});
        else
          out.push_back({reinterpret_cast<size_t>(gathered) + static_cast<size_t>(msg.slot0) * bytes, bytes});
      },
      stream);
  if (rc) return rc;
  B200_CUDA_OK(cudaEventRecord(cm->ev_rest, cm->stream));
  B200_CUDA_OK(cudaStreamWaitEvent(stream, cm->ev_rest, 0));
  return B200TRI_OK;
}

// ---------------------------------------------------------------------------- tri-mult
extern "C" size_t b200tri_trimul_cp_workspace_bytes(const b200tri_comm* cm, int32_t n) {
  if (!cm || n <= 0 || n % cm->cols) return 0;
  TileDims d;
  if (tile_dims(cm, n, &d)) return 0;
  const size_t a = trimul_plan(cm, d, false).total, b = trimul_plan(cm, d, true).total;
  return (a > b ? a : b) + 1024;
}

extern "C" int b200tri_trimul_cp(b200tri_comm* cm, const b200tri_trimul_cp_args* a, b200tri_stream_t stream_) {
  int rc = check_comm(cm, "trimul_cp");
  if (rc) return rc;
  B200_REQUIRE(a != nullptr && a->x && a->out, B200TRI_ERR_INVALID, "trimul_cp: null args, x or out");
  TileDims d;
  if ((rc = tile_dims(cm, a->n, &d))) return rc;
  const bool incoming = a->incoming != 0;
  const TrimulPlan pl = trimul_plan(cm, d, incoming);
  // workspace = NULL: the communicator's own exchange workspace (b200tri_comm_workspace), whose
  // peers' copies are mapped here, so tiles are copied through them instead of sent
  void* ws_ptr = a->workspace ? a->workspace : cm->ws;
  const size_t ws_have = a->workspace ? a->workspace_bytes : cm->ws_bytes;
  const bool pull = !a->workspace && !cm->peer_ws.empty();
  B200_REQUIRE(ws_ptr && ws_have >= pl.total, B200TRI_ERR_WORKSPACE,
               "trimul_cp: workspace of %zu bytes needed, got %zu", pl.total, ws_have);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(ws_ptr) & 1023) == 0, B200TRI_ERR_INVALID,
               "trimul_cp: workspace must be 1024-byte aligned");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(ws_ptr);
  const int R = cm->rows, C = cm->cols, m = cm->m, r = cm->r, c = cm->c;
  const int64_t n = d.n, n_r = d.n_r, n_c = d.n_c;
  (void)R;
  (void)C;

  // local projection of this rank's tile
  b200tri_trimul_project_args pa = {};
  pa.n_outer = pl.n_outer;
  pa.n_inner = pl.n_inner;
  pa.eps = a->eps;
  pa.x = a->x;
  pa.xs_outer = incoming ? 128 : n_c * 128;
  pa.xs_inner = incoming ? n_c * 128 : 128;
  if (a->mask) {
    pa.mask = a->mask + (static_cast<int64_t>(r) * n_r * n + static_cast<int64_t>(c) * n_c);
    pa.ms_outer = incoming ? 1 : n;
    pa.ms_inner = incoming ? n : 1;
  }
  pa.norm_in_scale = a->norm_in_scale;
  pa.norm_in_bias = a->norm_in_bias;
  pa.p_in = a->p_in;
  pa.g_in = a->g_in;
  pa.a = ws + pl.a_loc;
  pa.b = ws + pl.b_loc;
  pa.ld = pl.ld;
  pa.chan_stride = static_cast<int64_t>(pl.rpb) * pl.ld;
  pa.block_stride = static_cast<int64_t>(128) * pl.rpb * pl.ld;
  pa.rows_per_block = pl.rpb;
  pa.workspace = ws + pl.proj;
  pa.workspace_bytes = b200tri_trimul_project_workspace_bytes();
  log_launch(cm, B200TRI_CP_EVENT_PROJECT, -1, pa.n_outer, pa.n_inner, static_cast<uint8_t*>(pa.a) - ws,
             static_cast<uint8_t*>(pa.b) - ws, 0, 0);
  if (!cm->dry && (rc = b200tri_trimul_project(&pa, stream_))) return rc;

  // Exchange and contraction, in row chunks: the output rows of the tile are cut into G chunks
  // (k_split per n_c-row block); group g of the exchange carries chunk g of every `a` message
  // (group 0 all `b` messages as well) and fences the contraction of output chunk g alone, so all
  // but the last chunk are contracted while later groups travel. Channel-major data sits in
  // 64-row blocks of rb_bytes each, so a row chunk of a message is one contiguous piece.
  const size_t blk_bytes = pl.blk * 2;
  int k_split = 1;
  if (cm->world > 1 && pl.rpb == 64)
    for (k_split = m >= 4 ? 1 : 4 / m; k_split > 1 && (n_c % k_split || (n_c / k_split) % 128); k_split /= 2) {
    }
  // Which operand travels whole in the first group: the one the busiest rank sends less of. On a
  // square grid an outgoing rank sends one `a` tile but up to two `b` tiles, so there `a` goes
  // first and `b` is chunked: the chunks are then output COLUMNS (rows of `b`), a multiple of the
  // contraction's 256-column tile wide. Everywhere else (`a` panels are the larger ones) the
  // chunks are output rows, as described above.
  bool by_cols = false;
  if (!incoming && m == 1 && cm->world > 1 && pl.rpb == 64)
    for (int k = 4; k >= 2 && !by_cols; --k)
      if (n_c % k == 0 && (n_c / k) % 256 == 0) {
        by_cols = true;
        k_split = k;
      }
  const int G = m * k_split;
  const int64_t h = n_c / k_split;  // rows (or columns) per chunk
  const size_t rb_bytes = static_cast<size_t>(128) * 64 * pl.ld * 2;
  auto chunk_off = [&](int q) { return k_split > 1 ? static_cast<size_t>(q * h / 64) * rb_bytes : 0; };
  const size_t chunk_bytes = k_split > 1 ? static_cast<size_t>(h / 64) * rb_bytes : blk_bytes;
  CP_CUDA(cm, cudaEventRecord(cm->ev_ready, stream));
  CP_CUDA(cm, cudaStreamWaitEvent(cm->stream, cm->ev_ready, 0));
  const std::vector<Msg> msgs =
      build_plan(Grid{cm->rows, cm->cols, m}, incoming ? B200TRI_CP_TRIMUL_INCOMING : B200TRI_CP_TRIMUL_OUTGOING);
  for (int g = 0; g < G; ++g) {
    const int s = g / k_split, q = g % k_split;  // n_c-row block and chunk inside it
    rc = post_exchange(
        cm, ws, pull, msgs,
        [&](const Msg& msg) {
          if (by_cols) return msg.what == WHAT_A ? g == 0 : true;
          return msg.what == WHAT_B ? g == 0 : (!incoming || msg.slot0 == s);
        },
        [&](const Msg& msg, bool send, int who, std::vector<Piece>& out) {
          if (msg.what == WHAT_B) {
            const size_t off = by_cols ? chunk_off(g) : 0, bytes = by_cols ? chunk_bytes : blk_bytes;
            if (send) {
              const size_t b_loc = incoming ? pl.b_all + blk_bytes * (who / cm->cols) : pl.b_loc;
              out.push_back({b_loc + (msg.block < 0 ? 0 : blk_bytes * msg.block) + off, bytes});
            } else {
              out.push_back({pl.b_all + blk_bytes * msg.slot0 + off, bytes});
            }
            return;
          }
          if (by_cols) {  // the whole tile (m = 1: one block)
            out.push_back({pl.a_all + blk_bytes * (send ? who % cm->cols : msg.slot0), blk_bytes});
            return;
          }
          // `a`: the sender's local array has the receiver slot's layout; outgoing messages span
          // the m blocks of the tile (chunk g of all its rows), incoming ones one block (chunk q)
          size_t base;
          if (!incoming)
            base = pl.a_all + blk_bytes * m * (send ? who % cm->cols : msg.slot0) + blk_bytes * s;
          else
            base = send ? pl.a_loc : pl.a_all + blk_bytes * (static_cast<size_t>(msg.slot0) * cm->rows + msg.slot1);
          out.push_back({base + chunk_off(q), chunk_bytes});
        },
        stream, g == 0 && chunk_bytes < blk_bytes ? (by_cols ? WHAT_A : WHAT_B) : -1);
    if (rc) return rc;
    CP_CUDA(cm, cudaEventRecord(g + 1 < G ? cm->ev_part[g] : cm->ev_rest, cm->stream));
  }

  // one contraction launch per output chunk walks all k-sources (fp32 accumulation on chip)
  const int64_t t_chan = static_cast<int64_t>(pl.t_rpb) * pl.ldt;
  const int64_t t_row = pl.rpb == 64 ? static_cast<int64_t>(128) * pl.ldt : pl.ldt;
  for (int g = 0; g < G; ++g) {
    const int s = g / k_split, q = g % k_split;
    const bool last = g + 1 == G;
    CP_CUDA(cm, cudaStreamWaitEvent(stream, last ? cm->ev_rest : cm->ev_part[g], 0));
    b200tri_trimul_contract_args ca = {};
    ca.n_i = static_cast<int32_t>(by_cols ? n_r : h);
    ca.n_j = static_cast<int32_t>(by_cols ? h : n_c);
    ca.n_k = pl.n_k;
    ca.n_src = pl.n_src;
    if (by_cols) {
      ca.a = ws + pl.a_all;
      ca.a_src_stride = static_cast<int64_t>(pl.blk);
    } else if (!incoming) {
      ca.a = ws + pl.a_all + blk_bytes * s + chunk_off(q);
      ca.a_src_stride = static_cast<int64_t>(pl.blk) * m;
    } else {
      ca.a = ws + pl.a_all + blk_bytes * (static_cast<size_t>(s) * cm->rows) + chunk_off(q);
      ca.a_src_stride = static_cast<int64_t>(pl.blk);
    }
    ca.b = ws + pl.b_all + (by_cols ? chunk_off(g) : 0);
    ca.b_src_stride = static_cast<int64_t>(pl.blk);
    ca.a_ld = ca.b_ld = pl.ld;
    ca.a_chan_stride = ca.b_chan_stride = static_cast<int64_t>(pl.rpb) * pl.ld;
    ca.out_bf16 = by_cols ? ws + pl.t + static_cast<size_t>(2) * g * h
                          : ws + pl.t + static_cast<size_t>(2) * (static_cast<size_t>(s) * n_c + static_cast<size_t>(q) * h) * t_row;
    ca.out_ld = pl.ldt;
    ca.out_chan_stride = t_chan;
    ca.a_rows_per_block = ca.b_rows_per_block = pl.rpb;
    ca.out_rows_per_block = pl.t_rpb;
    ca.a_block_stride = ca.b_block_stride = static_cast<int64_t>(128) * pl.rpb * pl.ld;
    ca.out_block_stride = static_cast<int64_t>(128) * pl.t_rpb * pl.ldt;
    // later groups travel during these launches: leave their token kernels somewhere to run
    b200::SmReserve room(last ? 0 : cm->sm_reserve);
    log_launch(cm, B200TRI_CP_EVENT_CONTRACT, g, ca.n_i, ca.n_j, static_cast<const uint8_t*>(ca.a) - ws,
               static_cast<const uint8_t*>(ca.b) - ws, static_cast<uint8_t*>(ca.out_bf16) - ws, ca.a_src_stride * 2);
    if (!cm->dry && (rc = b200tri_trimul_contract(&ca, stream_))) return rc;

    // output stage of the same rows (or columns): it is local to a pair
    const int64_t row0 = by_cols ? 0 : static_cast<int64_t>(s) * n_c + static_cast<int64_t>(q) * h;
    const int64_t col0 = by_cols ? static_cast<int64_t>(g) * h : 0;
    const size_t pair0 = static_cast<size_t>(2) * (row0 * n_c + col0) * 128;  // byte offset of pair (row0, col0) in the tile
    b200tri_trimul_finish_args fa = {};
    fa.n_i = static_cast<int32_t>(by_cols ? n_r : h);
    fa.n_j = static_cast<int32_t>(by_cols ? h : n_c);
    fa.eps = a->eps;
    fa.t = ws + pl.t + static_cast<size_t>(2) * (row0 * t_row + col0);
    fa.t_ld = pl.ldt;
    fa.t_chan_stride = t_chan;
    fa.t_rows_per_block = pl.t_rpb;
    fa.t_block_stride = static_cast<int64_t>(128) * pl.t_rpb * pl.ldt;
    fa.x = static_cast<const uint8_t*>(a->x) + pair0;
    fa.xs_i = n_c * 128;
    fa.xs_j = 128;
    fa.norm_in_scale = a->norm_in_scale;
    fa.norm_in_bias = a->norm_in_bias;
    fa.norm_out_scale = a->norm_out_scale;
    fa.norm_out_bias = a->norm_out_bias;
    fa.p_out = a->p_out;
    fa.g_out = a->g_out;
    fa.residual = a->residual ? static_cast<const uint8_t*>(a->residual) + pair0 : nullptr;
    fa.out = static_cast<uint8_t*>(a->out) + pair0;
    fa.os_i = n_c * 128;
    fa.os_j = 128;
    fa.workspace = ws + pl.fin;
    fa.workspace_bytes = b200tri_trimul_finish_workspace_bytes();
    log_launch(cm, B200TRI_CP_EVENT_OUTPUT, g, fa.n_i, fa.n_j, static_cast<const uint8_t*>(fa.t) - ws, 0, 0,
               static_cast<uint8_t*>(fa.out) - static_cast<uint8_t*>(a->out));
    if (!cm->dry && (rc = b200tri_trimul_finish(&fa, stream_))) return rc;
  }
  return B200TRI_OK;
}

// ---------------------------------------------------------------------------- dry run
namespace {
// a communicator that exists on the host only: grid coordinates, fake non-null workspaces
void fake_comm(b200tri_comm* cm, int rows, int cols, int rank, int push, std::vector<b200tri_cp_event>* log) {
  cm->world = rows * cols;
  cm->rank = rank;
  cm->rows = rows;
  cm->cols = cols;
  cm->m = cols / rows;
  cm->r = rank / cols;
  cm->c = rank % cols;
  cm->push = push != 0;
  cm->dry = log;
  cm->ws = reinterpret_cast<void*>(static_cast<uintptr_t>(1) << 40);  // never dereferenced
  cm->ws_bytes = static_cast<size_t>(1) << 46;
  cm->peer_ws.assign(cm->world, cm->ws);
}
}  // namespace

extern "C" int b200tri_cp_dry_run(int32_t rows, int32_t cols, int32_t rank, int32_t n, int32_t op, int32_t push,
                                  b200tri_cp_event* out, int32_t capacity) {
  if (b200::check_grid(rows * cols, rows, cols)) return -1;
  if (rank < 0 || rank >= rows * cols || n <= 0 || n % cols || op < B200TRI_CP_TRIMUL_OUTGOING ||
      op > B200TRI_CP_TRIATT_ENDING) {
    b200::set_error("cp_dry_run: bad rank, token count or op");
    return -1;
  }
  std::vector<b200tri_cp_event> log;
  b200tri_comm cm;
  fake_comm(&cm, rows, cols, rank, push, &log);
  uint8_t* tile = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(1) << 50);  // stands for x and out; never dereferenced
  int rc;
  if (op <= B200TRI_CP_TRIMUL_INCOMING) {
    b200tri_trimul_cp_args a = {};
    a.n = n;
    a.incoming = op == B200TRI_CP_TRIMUL_INCOMING;
    a.eps = 1e-5f;
    a.x = tile;
    a.out = tile;
    rc = b200tri_trimul_cp(&cm, &a, nullptr);
  } else {
    b200tri_triatt_cp_args a = {};
    a.n = n;
    a.starting = op == B200TRI_CP_TRIATT_STARTING;
    a.heads = 4;
    a.head_dim = 32;
    a.eps = 1e-5f;
    a.inf = 1e9f;
    a.x = tile;
    a.out = tile;
    rc = b200tri_triatt_cp(&cm, &a, nullptr);
  }
  cm.peer_ws.clear();
  cm.ws = nullptr;
  if (rc) return -1;
  if (out)
    for (size_t i = 0; i < log.size() && static_cast<int32_t>(i) < capacity; ++i) out[i] = log[i];
  return static_cast<int>(log.size());
}

extern "C" int b200tri_cp_layout(int32_t rows, int32_t cols, int32_t rank, int32_t n, int32_t op, int64_t* out) {
  if (b200::check_grid(rows * cols, rows, cols)) return -1;
  if (!out || rank < 0 || rank >= rows * cols || n <= 0 || n % cols || op < B200TRI_CP_TRIMUL_OUTGOING ||
      op > B200TRI_CP_TRIATT_ENDING) {
    b200::set_error("cp_layout: bad rank, token count, op or buffer");
    return -1;
  }
  b200tri_comm cm;
  fake_comm(&cm, rows, cols, rank, 1, nullptr);
  cm.peer_ws.clear();
  cm.ws = nullptr;
  b200::TileDims d;
  if (b200::tile_dims(&cm, n, &d)) return -1;
  for (int i = 0; i < 16; ++i) out[i] = 0;
  if (op <= B200TRI_CP_TRIMUL_INCOMING) {
    const b200::TrimulPlan pl = b200::trimul_plan(&cm, d, op == B200TRI_CP_TRIMUL_INCOMING);
    const int64_t v[8] = {(int64_t)pl.a_all, (int64_t)pl.a_loc, (int64_t)pl.b_all, (int64_t)pl.b_loc, (int64_t)pl.blk * 2,
                          op == B200TRI_CP_TRIMUL_INCOMING ? 1 : cm.m, (int64_t)pl.t, (int64_t)pl.total};
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  } else {
    const b200::TriattPlan pl = b200::triatt_plan(&cm, d, op == B200TRI_CP_TRIATT_STARTING);
    const int64_t v[11] = {(int64_t)pl.q, (int64_t)pl.k_all, (int64_t)pl.vt_all, (int64_t)pl.bias_loc, (int64_t)pl.bias_all,
                           (int64_t)pl.k_tile, (int64_t)pl.vt_tile, (int64_t)pl.bias_tile, pl.tiles, pl.own, (int64_t)pl.total};
    for (int i = 0; i < 11; ++i) out[i] = v[i];
  }
  return 0;
}

// ---------------------------------------------------------------------------- tri-attn
extern "C" size_t b200tri_triatt_cp_workspace_bytes(const b200tri_comm* cm, int32_t n) {
  if (!cm || n <= 0 || n % cm->cols) return 0;
  TileDims d;
  if (tile_dims(cm, n, &d)) return 0;
  const size_t a = triatt_plan(cm, d, true).total, b = triatt_plan(cm, d, false).total;
  return (a > b ? a : b) + 1024;
}

extern "C" int b200tri_triatt_cp(b200tri_comm* cm, const b200tri_triatt_cp_args* a, b200tri_stream_t stream_) {
  int rc = check_comm(cm, "triatt_cp");
  if (rc) return rc;
  B200_REQUIRE(a != nullptr && a->x && a->out, B200TRI_ERR_INVALID, "triatt_cp: null args, x or out");
  B200_REQUIRE(a->heads == 4 && a->head_dim == 32, B200TRI_ERR_UNSUPPORTED,
               "triatt_cp: built for 4 heads x 32 (got %d x %d)", a->heads, a->head_dim);
  TileDims d;
  if ((rc = tile_dims(cm, a->n, &d))) return rc;
  const bool starting = a->starting != 0;
  const TriattPlan pl = triatt_plan(cm, d, starting);
  B200_REQUIRE(pl.tiles <= 1 + 7, B200TRI_ERR_UNSUPPORTED, "triatt_cp: at most 8 key tiles per ring (got %d)", pl.tiles);
  void* ws_ptr = a->workspace ? a->workspace : cm->ws;
  const size_t ws_have = a->workspace ? a->workspace_bytes : cm->ws_bytes;
  const bool pull = !a->workspace && !cm->peer_ws.empty();
  B200_REQUIRE(ws_ptr && ws_have >= pl.total, B200TRI_ERR_WORKSPACE,
               "triatt_cp: workspace of %zu bytes needed, got %zu", pl.total, ws_have);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(ws_ptr) & 1023) == 0, B200TRI_ERR_INVALID,
               "triatt_cp: workspace must be 1024-byte aligned");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(ws_ptr);
  const int m = cm->m, r = cm->r, c = cm->c;
  const int64_t n = d.n, n_r = d.n_r, n_c = d.n_c;
  const int64_t xs_o = starting ? n_c * 128 : 128, xs_i = starting ? 128 : n_c * 128;

  b200tri_triatt_project_args pa = {};
  pa.n_outer = pl.n_outer;
  pa.n_inner = pl.n_inner;
  pa.heads = a->heads;
  pa.head_dim = a->head_dim;
  pa.eps = a->eps;
  pa.x = a->x;
  pa.xs_outer = xs_o;
  pa.xs_inner = xs_i;
  pa.norm_scale = a->norm_scale;
  pa.norm_bias = a->norm_bias;
  pa.w_q = a->w_q;
  pa.w_k = a->w_k;
  pa.w_v = a->w_v;
  pa.w_bias = a->w_bias;
  pa.q = ws + pl.q;
  pa.k = ws + pl.k_all + pl.k_tile * pl.own;
  pa.vt = ws + pl.vt_all + pl.vt_tile * pl.own;
  pa.bias = ws + pl.bias_loc;
  pa.ld = pl.ld;
  pa.bias_head_stride = static_cast<int64_t>(pl.n_outer) * pl.ld;
  pa.workspace = ws + pl.proj;
  pa.workspace_bytes = b200tri_triatt_project_workspace_bytes();
  log_launch(cm, B200TRI_CP_EVENT_PROJECT, -1, pa.n_outer, pa.n_inner, static_cast<uint8_t*>(pa.q) - ws,
             static_cast<uint8_t*>(pa.k) - ws, static_cast<uint8_t*>(pa.vt) - ws, static_cast<uint8_t*>(pa.bias) - ws);
  if (!cm->dry && (rc = b200tri_triatt_project(&pa, stream_))) return rc;

  // Two groups on the exchange stream: the bias chunks (small; even the own key tile's bias
  // may live on another rank) fence the first core launch, the peers' K/V tiles only the
  // second one, so they travel while the own key tile is computed.
  CP_CUDA(cm, cudaEventRecord(cm->ev_ready, stream));
  CP_CUDA(cm, cudaStreamWaitEvent(cm->stream, cm->ev_ready, 0));
  const std::vector<Msg> msgs =
      build_plan(Grid{cm->rows, cm->cols, m}, starting ? B200TRI_CP_TRIATT_STARTING : B200TRI_CP_TRIATT_ENDING);
  const size_t head_rows = static_cast<size_t>(pl.n_outer) * pl.ld * 2;  // one head of the sender's bias
  const size_t qhead = static_cast<size_t>(pl.n_q) * pl.ld * 2;          // one head of a received bias tile
  const size_t chunk = static_cast<size_t>(n_c) * pl.ld * 2;             // n_c bias rows
  auto views = [&](const Msg& msg, bool send, int who, std::vector<Piece>& out) {
    if (msg.what == WHAT_KV) {  // the sender's own key tile sits in its own slot
      const int slot = send ? (starting ? who % cm->cols : who / cm->cols) : msg.slot0;
      out.push_back({pl.k_all + pl.k_tile * slot, pl.k_tile});
      out.push_back({pl.vt_all + pl.vt_tile * slot, pl.vt_tile});
      return;
    }
    for (int h = 0; h < 4; ++h) {
      if (starting) {  // row block of the sender's bias -> the whole bias of one key tile
        if (send)
          out.push_back({pl.bias_loc + head_rows * h + chunk * msg.block, chunk});
        else
          out.push_back({pl.bias_all + pl.bias_tile * msg.slot0 + qhead * h, chunk});
      } else {  // the sender's whole bias -> one query block of one key tile
        if (send)
          out.push_back({pl.bias_loc + head_rows * h, chunk});
        else
          out.push_back({pl.bias_all + pl.bias_tile * msg.slot0 + qhead * h + chunk * msg.slot1, chunk});
      }
    }
  };
  if ((rc = post_exchange(cm, ws, pull, msgs, [](const Msg& x) { return x.what == WHAT_BIAS; }, views, stream))) return rc;
  CP_CUDA(cm, cudaEventRecord(cm->ev_first, cm->stream));
  // The peers' key tiles travel in groups of 1, 2, 4 tiles (in the order they are walked), each
  // fencing its own core launch: the first peer tile is computed while the next two arrive, and
  // so on, at the price of one spill of the running state per extra launch.
  const bool grouped = pl.n_inner % 64 == 0;
  auto group_of = [&](const Msg& msg) {  // of a K/V message, seen from its receiver
    const int own = starting ? msg.dst % cm->cols : msg.dst / cm->cols;
    const int idx = (msg.slot0 - own + pl.tiles) % pl.tiles;  // position in the receiver's walk (>= 1)
    return !grouped ? 0 : idx < 2 ? 0 : idx < 4 ? 1 : 2;
  };
  const int n_groups = !grouped || pl.tiles <= 2 ? 1 : pl.tiles <= 4 ? 2 : 3;
  for (int g = 0; g < n_groups; ++g) {
    if ((rc = post_exchange(cm, ws, pull, msgs, [&](const Msg& x) { return x.what == WHAT_KV && group_of(x) == g; },
                            views, stream)))
      return rc;
    CP_CUDA(cm, cudaEventRecord(g + 1 < n_groups ? cm->ev_part[g] : cm->ev_rest, cm->stream));
  }

  // key tiles: the own one first, then the peers' in rotated order (every sender serves a
  // different receiver at each position), all of them in one resumed launch
  b200tri_triatt_core_args tiles[8] = {};
  for (int idx = 0; idx < pl.tiles; ++idx) {
    const int t = (pl.own + idx) % pl.tiles;
    b200tri_triatt_core_args& ca = tiles[idx];
    ca.n_i = pl.n_outer;
    ca.n_j = pl.n_q;
    ca.n_k = pl.n_inner;
    ca.heads = a->heads;
    ca.head_dim = a->head_dim;
    ca.q = ws + pl.q;
    ca.k = ws + pl.k_all + pl.k_tile * t;
    ca.vt = ws + pl.vt_all + pl.vt_tile * t;
    ca.v_ld = pl.ld;
    ca.bias = ws + pl.bias_all + pl.bias_tile * t;
    ca.bias_ld = pl.ld;
    ca.bias_head_stride = static_cast<int64_t>(pl.n_q) * pl.ld;
    if (a->mask) {
      if (starting) {  // rows I_r, keys K_t
        ca.mask = a->mask + (static_cast<int64_t>(r) * n_r * n + static_cast<int64_t>(t) * n_c);
        ca.ms_i = n;
        ca.ms_k = 1;
      } else {  // rows J_c, keys I_t of the transposed mask
        ca.mask = a->mask + (static_cast<int64_t>(t) * n_r * n + static_cast<int64_t>(c) * n_c);
        ca.ms_i = 1;
        ca.ms_k = n;
      }
    }
    ca.inf = a->inf;
    ca.o = ws + pl.o;
    ca.row_max = reinterpret_cast<float*>(ws + pl.rmax);
    ca.row_sum = reinterpret_cast<float*>(ws + pl.rsum);
    ca.acc_o = reinterpret_cast<float*>(ws + pl.acc);
    ca.workspace = ws + pl.core;
    ca.workspace_bytes = b200tri_triatt_core_multi_workspace_bytes(pl.n_outer, pl.n_inner, pl.tiles);
  }
  // dry-run log of one core launch: walk positions [lo, hi) of the key-tile order
  auto log_core = [&](int launch, int lo, int hi) {
    for (int idx = lo; idx < hi; ++idx)
      log_launch(cm, B200TRI_CP_EVENT_CORE_TILE, launch, idx, (pl.own + idx) % pl.tiles,
                 static_cast<const uint8_t*>(tiles[idx].k) - ws, static_cast<const uint8_t*>(tiles[idx].vt) - ws,
                 static_cast<const uint8_t*>(tiles[idx].bias) - ws, 0);
  };
  CP_CUDA(cm, cudaStreamWaitEvent(stream, cm->ev_first, 0));
  tiles[0].unnormalized = pl.tiles > 1;
  {
    // the peers' key tiles travel during this launch: leave their token kernels somewhere to run
    b200::SmReserve room(pl.tiles > 1 ? cm->sm_reserve : 0);
    log_core(0, 0, 1);
    if (!cm->dry && (rc = b200tri_triatt_core(&tiles[0], stream_))) return rc;
  }
  if (pl.tiles > 1) {
    if (grouped) {
      for (int g = 0, lo = 1; g < n_groups; ++g) {
        const int hi = std::min(pl.tiles, 2 << g);  // walk positions [lo, hi)
        const bool last = g + 1 == n_groups;
        CP_CUDA(cm, cudaStreamWaitEvent(stream, last ? cm->ev_rest : cm->ev_part[g], 0));
        tiles[lo].resume = 1;
        tiles[lo].unnormalized = !last;
        b200::SmReserve room(last ? 0 : cm->sm_reserve);
        log_core(g + 1, lo, hi);
        if (!cm->dry && (rc = b200tri_triatt_core_multi(&tiles[lo], hi - lo, stream_))) return rc;
        lo = hi;
      }
    } else {  // ragged key tiles: one launch each, the state carried in acc_o
      CP_CUDA(cm, cudaStreamWaitEvent(stream, cm->ev_rest, 0));
      for (int idx = 1; idx < pl.tiles; ++idx) {
        tiles[idx].resume = 1;
        tiles[idx].unnormalized = idx + 1 < pl.tiles;
        log_core(idx, idx, idx + 1);
        if (!cm->dry && (rc = b200tri_triatt_core(&tiles[idx], stream_))) return rc;
      }
    }
  }

  b200tri_triatt_finish_args fa = {};
  fa.n_outer = pl.n_outer;
  fa.n_inner = pl.n_inner;
  fa.eps = a->eps;
  fa.o = ws + pl.o;
  fa.x = a->x;
  fa.xs_outer = xs_o;
  fa.xs_inner = xs_i;
  fa.norm_scale = a->norm_scale;
  fa.norm_bias = a->norm_bias;
  fa.w_g = a->w_g;
  fa.w_o = a->w_o;
  fa.residual = a->residual;
  fa.out = a->out;
  fa.os_outer = xs_o;
  fa.os_inner = xs_i;
  fa.workspace = ws + pl.fin;
  fa.workspace_bytes = b200tri_triatt_finish_workspace_bytes();
  if (cm->dry) return B200TRI_OK;
  return b200tri_triatt_finish(&fa, stream_);
}
