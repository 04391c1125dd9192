// Host-side stress of the native core, meant to be built with -fsanitize=address,undefined and with
// -fsanitize=thread (tests/test_sanitizers.py does both):
//   1. page pool: random allocate / release with the accounting invariants checked at every step;
//   2. controller inside the virtual-time cluster simulator: a bursty trace with live scaling and a replica
//      failure in the middle; every request must finish, no KV block may leak;
//   3. the device protocols, emulated with CPU threads on std::atomic (what the kernels do with
//      st.release / ld.acquire and tickets):
//        a. unit copy: producer writes a unit, then release-adds 1 to its flag; consumers acquire-poll with a
//           bounded spin, read the unit, and the single consumer that owns the flag resets it;
//        b. split-K tickets: every contributor stores its partial, takes a ticket (acq_rel); the last one sums the
//           partials in index order and resets the ticket.
//        c. one-kernel all-reduce: blocks of the same index on all ranks rendezvous through per-block counters in two
//           alternating parities; slots are reused every second call without any other synchronisation.
//        d. KV push of a partial migration: page ids and a tag published by the destination, two sources pushing
//           disjoint layer ranges into the same transfer slot, growing per-layer arrival counters.
//      ThreadSanitizer checks that the data accesses are ordered by those atomics.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "runtime/kv_pool.h"
#include "sim/cluster_sim.h"
#include "sim/trace.h"
#include "util/pbwire.h"

using namespace blitz;

#define CHECK(cond)                                                            \
  do {                                                                         \
    if (!(cond)) {                                                             \
      std::fprintf(stderr, "CHECK failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__); \
      std::exit(1);                                                            \
    }                                                                          \
  } while (0)

static void pool_fuzz() {
  PagePool pool(257, 16);
  std::mt19937 rng(5);
  std::vector<std::vector<int32_t>> held;
  int used = 0;
  for (int it = 0; it < 20000; ++it) {
    if (held.empty() || rng() % 3) {
      const int n = static_cast<int>(rng() % 9);
      std::vector<int32_t> got;
      const bool ok = pool.allocate(n, got);
      CHECK(ok == (n <= 257 - used));
      if (ok) {
        for (int32_t p : got) CHECK(pool.is_used(p));
        used += n;
        held.push_back(std::move(got));
      }
    } else {
      const size_t i = rng() % held.size();
      pool.release(held[i]);
      used -= static_cast<int>(held[i].size());
      held.erase(held.begin() + static_cast<long>(i));
    }
    CHECK(pool.used_pages() == used && pool.free_pages() == 257 - used);
  }
  bool threw = false;
  try {
    pool.release(std::vector<int32_t>(2, 0));   // page 0 is not held (everything was released or never handed out twice)
  } catch (const std::logic_error&) {
    threw = true;
  }
  CHECK(threw);
}

// The wire reader takes whatever bytes a worker sends: valid responses round-trip, and truncated, bit-flipped or random
// bytes either parse or raise, without a read outside the buffer (which the address sanitizer would report).
static void wire_fuzz() {
  std::mt19937 rng(11);
  PagePool pool(64, 16);
  Batch b(1, &pool);
  std::vector<SeqSpec> specs;
  for (int i = 0; i < 5; ++i) {
    SeqSpec s;
    s.id = 1000u + i;
    s.prompt = {1, 2, 3};
    s.max_new_tokens = 1 + i % 2;
    s.eos_token = 7;
    s.ignore_eos = false;
    specs.push_back(s);
  }
  CHECK(b.add_prompts(specs));
  b.mark_prefilled();
  const std::vector<int32_t> toks = {5, 6, 7, 8, 9};
  b.append_tokens(toks, false);
  const std::string good = b.encode_generations(toks);
  const pbwire::Generations g = pbwire::parse_generations(good);
  CHECK(g.request_ids.size() == 5 && g.tokens == toks && g.request_ids[4] == 1004u);
  CHECK(g.finished[0] && g.reasons[0] == 0 && !g.finished[1] && g.reasons[1] == -1 && g.finished[2] && g.reasons[2] == 1);
  size_t parsed = 0, refused = 0;
  for (int it = 0; it < 20000; ++it) {
    std::string m = good;
    switch (it % 4) {
      case 0: m.resize(rng() % (good.size() + 1)); break;
      case 1: for (int k = 0; k < 3; ++k) m[rng() % m.size()] = static_cast<char>(rng()); break;
      case 2: m.assign(rng() % 64, '\0'); for (auto& c : m) c = static_cast<char>(rng()); break;
      default: m.insert(rng() % m.size(), 1, static_cast<char>(rng())); break;
    }
    try {
      const pbwire::Generations x = pbwire::parse_generations(m);
      CHECK(x.request_ids.size() == x.tokens.size() && x.tokens.size() == x.finished.size() && x.finished.size() == x.reasons.size());
      ++parsed;
    } catch (const std::invalid_argument&) {
      ++refused;
    }
  }
  CHECK(parsed > 0 && refused > 0);
  b.clear();
}

static void controller_sim() {
  ControllerConfig cc;
  cc.num_ranks = 6;
  cc.tp = 1;
  cc.init_states = {"Prefill", "Decode", "Inactive", "Inactive", "Inactive", "Inactive"};
  cc.features = "impl_blitz,impl_nvl,impl_live";
  CostModel cm;
  TraceSpec ts;
  ts.phases = {{0.0, 4.0}, {3.0, 40.0}, {8.0, 4.0}};
  ts.cv = 2.0;
  ts.duration = 12.0;
  ts.input.a = 400;
  ts.output.a = 24;
  ts.seed = 9;
  const std::vector<TraceItem> trace = generate_trace(ts);
  {
    ClusterSim sim(cc, cm);
    const SimReport rep = sim.run(trace, 0.001, 120.0);
    CHECK(rep.submitted == trace.size() && rep.completed == rep.submitted && rep.failed == 0);
    CHECK(rep.leftover_blocks == 0);
  }
  {
    ClusterSim sim(cc, cm);
    const SimReport rep = sim.run(trace, 0.001, 120.0, /*kill_replica=*/1, /*kill_at=*/5.0);
    CHECK(rep.submitted == trace.size() && rep.completed + rep.failed == rep.submitted);
    CHECK(rep.leftover_blocks == 0);
  }
  for (int tp : {1, 2}) {
    // failures of every replica in turn, clients that leave, several migrations in flight, tensor-parallel replicas
    ControllerConfig c2 = cc;
    c2.tp = tp;
    c2.num_ranks = 6 * tp;
    c2.init_states.clear();
    for (const char* st : {"Prefill", "Decode", "Prefill", "Inactive", "Inactive", "Inactive"})
      for (int k = 0; k < tp; ++k) c2.init_states.push_back(st);
    c2.max_incoming_migrations = 3;
    c2.quarantine_ms = 300;
    for (const char* feats : {"impl_blitz,impl_nvl,impl_live", "impl_blitz,impl_nvl,impl_live,migrate_progressive"}) {
      c2.features = feats;   // the second set places a batch on its decode replica when its prefill is issued
      for (int victim = 0; victim < 3; ++victim) {
        ClusterSim sim(c2, cm);
        const SimReport rep = sim.run(trace, 0.001, 120.0, victim, 4.0 + victim, /*gone_every=*/4);
        CHECK(rep.submitted == trace.size() && rep.completed + rep.failed + rep.gone_in_queue == rep.submitted);
        CHECK(rep.leftover_blocks == 0);
      }
    }
  }
}

// ---- 3a: unit copy with per-unit flags -------------------------------------------------------------------
static void flag_protocol() {
  constexpr int kUnits = 64, kWords = 1024, kRounds = 20, kReaders = 3;
  std::vector<uint32_t> buf(static_cast<size_t>(kUnits) * kWords);
  std::vector<std::atomic<uint32_t>> flags(kUnits);
  std::atomic<int> readers_done{0};
  std::atomic<uint32_t> round_go{0};
  std::atomic<bool> failed{false};
  for (auto& f : flags) f.store(0);

  auto bounded_wait = [&](std::atomic<uint32_t>& f, uint32_t want) {
    const auto t0 = std::chrono::steady_clock::now();
    while (f.load(std::memory_order_acquire) < want) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) return false;
      std::this_thread::yield();
    }
    return true;
  };
  std::thread producer([&] {
    for (int r = 1; r <= kRounds; ++r) {
      // the flag owner re-armed every flag of the previous round before it let us go on
      if (!bounded_wait(round_go, static_cast<uint32_t>(r - 1))) { failed = true; return; }
      for (int u = 0; u < kUnits; ++u) {
        for (int w = 0; w < kWords; ++w) buf[static_cast<size_t>(u) * kWords + w] = static_cast<uint32_t>(r * 1000003 + u * 131 + w);
        flags[u].fetch_add(1, std::memory_order_release);
      }
    }
  });
  std::vector<std::thread> readers;
  for (int k = 0; k < kReaders; ++k)
    readers.emplace_back([&, k] {
      for (int r = 1; r <= kRounds; ++r) {
        for (int u = 0; u < kUnits; ++u) {
          if (!bounded_wait(flags[u], 1)) { failed = true; return; }
          for (int w = k; w < kWords; w += 97)
            if (buf[static_cast<size_t>(u) * kWords + w] != static_cast<uint32_t>(r * 1000003 + u * 131 + w)) failed = true;
        }
        // readers meet; reader 0 owns the flags: it re-arms them, then releases the producer into the next pass
        readers_done.fetch_add(1, std::memory_order_acq_rel);
        while (readers_done.load(std::memory_order_acquire) < kReaders * r) std::this_thread::yield();
        if (k == 0) {
          for (auto& f : flags) f.store(0, std::memory_order_relaxed);
          round_go.store(static_cast<uint32_t>(r), std::memory_order_release);
        } else {
          if (!bounded_wait(round_go, static_cast<uint32_t>(r))) { failed = true; return; }
        }
      }
    });
  producer.join();
  for (auto& t : readers) t.join();
  CHECK(!failed.load());
  // a flag nobody sets: the bounded wait gives up and reports it
  std::atomic<uint32_t> never{0};
  const auto t0 = std::chrono::steady_clock::now();
  while (never.load(std::memory_order_acquire) < 1 && std::chrono::steady_clock::now() - t0 < std::chrono::milliseconds(20)) {}
  CHECK(never.load() == 0);
}

// ---- 3b: split-K tickets ---------------------------------------------------------------------------------
static void ticket_protocol() {
  constexpr int kSplit = 4, kTiles = 32, kElems = 256, kLaunches = 30;
  std::vector<float> ws(static_cast<size_t>(kTiles) * kSplit * kElems);
  std::vector<float> out(static_cast<size_t>(kTiles) * kElems);
  std::vector<std::atomic<uint32_t>> tickets(kTiles);
  for (auto& t : tickets) t.store(0);
  for (int launch = 0; launch < kLaunches; ++launch) {
    std::vector<std::thread> ctas;
    for (int s = 0; s < kSplit; ++s)
      ctas.emplace_back([&, s] {
        for (int tile = 0; tile < kTiles; ++tile) {
          float* part = &ws[(static_cast<size_t>(tile) * kSplit + s) * kElems];
          for (int i = 0; i < kElems; ++i) part[i] = static_cast<float>((launch + 1) * (s + 1)) + 0.25f * static_cast<float>(i % 4);
          const uint32_t old = tickets[tile].fetch_add(1, std::memory_order_acq_rel);
          if (old == kSplit - 1) {
            tickets[tile].store(0, std::memory_order_relaxed);  // ready for the next launch
            for (int i = 0; i < kElems; ++i) {
              float acc = 0.f;
              for (int k = 0; k < kSplit; ++k) acc += ws[(static_cast<size_t>(tile) * kSplit + k) * kElems + i];
              out[static_cast<size_t>(tile) * kElems + i] = acc;
            }
          }
        }
      });
    for (auto& t : ctas) t.join();
    for (int tile = 0; tile < kTiles; ++tile)
      for (int i = 0; i < kElems; ++i)
        CHECK(out[static_cast<size_t>(tile) * kElems + i] == static_cast<float>((launch + 1) * 10) + static_cast<float>(i % 4));
    for (auto& t : tickets) CHECK(t.load() == 0);
  }
}

// ---- 3c: one-kernel all-reduce over peer memory, two parities -----------------------------------------------
// Rank r, block b (one thread each here) of call c: store its chunk of the local vector into slot [parity][r] of
// every rank, release-add 1 to counter [parity][r][b] on every rank, acquire-wait for counters [parity][s][b] of all
// sources on its own rank, sum the slots in rank order, re-arm the counters it consumed.  Calls alternate between
// two parities; a rank starts call c + 1 only when all its blocks have finished call c (stream order).  The claim
// under test: that alone orders a peer's next write into a slot after this rank's last read of it.
static void allreduce_protocol() {
  constexpr int kTp = 4, kBlocks = 4, kChunk = 64, kCalls = 200;
  constexpr int kN = kBlocks * kChunk;
  struct Rank {
    std::vector<float> slots;                       // [parity][src][n]
    std::vector<std::atomic<uint32_t>> flags;       // [parity][src][block]
    std::vector<float> out;
    std::atomic<int> blocks_done{0};
    Rank() : slots(2 * kTp * kN), flags(2 * kTp * kBlocks), out(kN) { for (auto& f : flags) f.store(0); }
  };
  std::vector<Rank> ranks(kTp);
  std::atomic<bool> failed{false};
  auto contribution = [](int call, int rank, int i) { return static_cast<float>((call % 17) * 64 + rank * 8 + (i % 5)); };
  std::vector<std::thread> threads;
  for (int r = 0; r < kTp; ++r)
    for (int b = 0; b < kBlocks; ++b)
      threads.emplace_back([&, r, b] {
        Rank& me = ranks[r];
        for (int c = 0; c < kCalls; ++c) {
          const int par = c & 1;
          for (int d = 0; d < kTp; ++d)
            for (int i = b * kChunk; i < (b + 1) * kChunk; ++i)
              ranks[d].slots[(static_cast<size_t>(par) * kTp + r) * kN + i] = contribution(c, r, i);
          for (int d = 0; d < kTp; ++d)
            ranks[d].flags[(static_cast<size_t>(par) * kTp + r) * kBlocks + b].fetch_add(1, std::memory_order_release);
          for (int s = 0; s < kTp; ++s) {
            auto& f = me.flags[(static_cast<size_t>(par) * kTp + s) * kBlocks + b];
            const auto t0 = std::chrono::steady_clock::now();
            while (f.load(std::memory_order_acquire) < 1) {
              if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(30)) { failed = true; return; }
              std::this_thread::yield();
            }
          }
          for (int i = b * kChunk; i < (b + 1) * kChunk; ++i) {
            float acc = 0.f, want = 0.f;
            for (int s = 0; s < kTp; ++s) {
              acc += me.slots[(static_cast<size_t>(par) * kTp + s) * kN + i];
              want += contribution(c, s, i);
            }
            me.out[i] = acc;
            if (acc != want) failed = true;
          }
          for (int s = 0; s < kTp; ++s)
            me.flags[(static_cast<size_t>(par) * kTp + s) * kBlocks + b].store(0, std::memory_order_relaxed);
          // end of the kernel on this rank: the next call starts when every block of this one has finished
          me.blocks_done.fetch_add(1, std::memory_order_acq_rel);
          while (me.blocks_done.load(std::memory_order_acquire) < kBlocks * (c + 1)) std::this_thread::yield();
        }
      });
  for (auto& t : threads) t.join();
  CHECK(!failed.load());
  for (auto& rk : ranks)
    for (auto& f : rk.flags) CHECK(f.load() == 0);
}

// ---- 3d: KV push into a transfer slot, two sources (partial migration) ------------------------------------------
// The destination publishes the page ids of the batch in its control slot, then release-stores the batch's tag.  Each
// source acquire-waits for the tag, reads the page ids, stores the KV of ITS layers (the new instance layers [0, k),
// the old instance layers [k, L)) into those pages and release-adds 1 to the per-layer arrival counter.  The
// destination acquire-waits until every layer's counter has reached the value it expects for this batch (the counters
// only grow; the destination keeps the expected values), uses the pages and moves on to the next batch in the same
// slot.  Every wait is bounded.
static void kv_push_protocol() {
  constexpr int kLayers = 8, kPages = 6, kPageWords = 128, kBatches = 150, kPool = 64;
  std::vector<uint32_t> pool(static_cast<size_t>(kLayers) * kPool * kPageWords);   // [layer][page][word]
  std::vector<int> page_ids(kPages);
  std::atomic<uint32_t> tag{0};
  std::vector<std::atomic<uint32_t>> arrived(kLayers);
  for (auto& a : arrived) a.store(0);
  std::atomic<bool> failed{false};
  auto wait_until = [&](auto pred) {
    const auto t0 = std::chrono::steady_clock::now();
    while (!pred()) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(30)) return false;
      std::this_thread::yield();
    }
    return true;
  };
  auto split_of = [](int batch) { return 1 + batch % (kLayers - 1); };   // k: first layer of the old instance's half
  auto word = [](int batch, int layer, int page, int w) { return static_cast<uint32_t>(batch * 7919 + layer * 131 + page * 17 + w); };
  auto source = [&](bool first_half) {
    for (int b = 1; b <= kBatches; ++b) {
      if (!wait_until([&] { return tag.load(std::memory_order_acquire) == static_cast<uint32_t>(b); })) { failed = true; return; }
      const int k = split_of(b);
      for (int l = first_half ? 0 : k; l < (first_half ? k : kLayers); ++l) {
        for (int p = 0; p < kPages; ++p)
          for (int w = 0; w < kPageWords; ++w)
            pool[(static_cast<size_t>(l) * kPool + page_ids[p]) * kPageWords + w] = word(b, l, p, w);
        arrived[l].fetch_add(1, std::memory_order_release);
      }
    }
  };
  std::thread newer(source, true), older(source, false);
  std::mt19937 rng(3);
  for (int b = 1; b <= kBatches; ++b) {
    for (int p = 0; p < kPages; ++p) page_ids[p] = (static_cast<int>(rng() % 9) * kPages + p) % kPool;   // distinct pages
    tag.store(static_cast<uint32_t>(b), std::memory_order_release);
    for (int l = 0; l < kLayers; ++l)
      if (!wait_until([&] { return arrived[l].load(std::memory_order_acquire) >= static_cast<uint32_t>(b); })) failed = true;
    if (failed) break;
    for (int l = 0; l < kLayers; ++l)
      for (int p = 0; p < kPages; ++p)
        for (int w = 0; w < kPageWords; w += 31)
          if (pool[(static_cast<size_t>(l) * kPool + page_ids[p]) * kPageWords + w] != word(b, l, p, w)) failed = true;
  }
  if (failed) tag.store(0xFFFFFFFFu, std::memory_order_release);
  newer.join();
  older.join();
  CHECK(!failed.load());
}

int main(int argc, char** argv) {
  const std::string what = argc > 1 ? argv[1] : "all";
  if (what == "all" || what == "pool") pool_fuzz();
  if (what == "all" || what == "wire") wire_fuzz();
  if (what == "all" || what == "sim") controller_sim();
  if (what == "all" || what == "flags") flag_protocol();
  if (what == "all" || what == "tickets") ticket_protocol();
  if (what == "all" || what == "allreduce") allreduce_protocol();
  if (what == "all" || what == "kvpush") kv_push_protocol();
  std::printf("core_stress %s: OK\n", what.c_str());
  return 0;
}
