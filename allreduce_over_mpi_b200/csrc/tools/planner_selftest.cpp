// Self-test of the host-only core, meant to be built with sanitizers:
//     g++ -std=c++17 -O1 -g -fsanitize=address,undefined planner_selftest.cpp -o t && ./t
//     g++ -std=c++17 -O1 -g -fsanitize=thread planner_selftest.cpp -o t -lpthread && ./t threads
// It builds the plan of every executable shape up to 24 ranks, runs the static race check and the
// snapshot executor against a double-precision sum, exercises the candidate enumerators and the
// cost models, checks the device tables (and that damaged ones are refused) and the heap allocator, and (argument "threads") runs the thread-per-rank executor with its flag protocol,
// including a silent rank that must produce time-outs rather than a hang.
// The reference has no sanitizer builds (its flags are -Wall -Wextra only, allreduce_over_mpi/CMakeLists.txt:5).
#include <sys/wait.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../planner/config.hpp"
#include "../planner/cost_model.hpp"
#include "../planner/cpu_executor.hpp"
#include "../planner/policy.hpp"
#include "../planner/proc_world.hpp"
#include "../runtime/dev_plan.hpp"
#include "../runtime/heap_alloc.hpp"
#include "../runtime/fd_channel.cpp"   // descriptor passing over abstract unix sockets: plain host code, compiled in here

static int fails = 0;
#define EXPECT(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); ++fails; } } while (0)

static void plans_and_snapshot() {
  int checked = 0;
  for (int n = 1; n <= 24; ++n)
    for (const ft::Shape& s : ft::executable_shapes(n)) {
      ft::Plan p = ft::build_plan(n, s);
      EXPECT(p.ok());
      EXPECT(ft::check_hazards(p).empty());
      for (uint64_t count : {1ull, 29ull, 257ull}) {
        std::vector<std::vector<double>> data(n, std::vector<double>(count));
        std::vector<double> want(count, 0.0);
        for (int r = 0; r < n; ++r)
          for (uint64_t i = 0; i < count; ++i) { data[r][i] = std::sin(r * 131 + i * 7) ; want[i] += data[r][i]; }
        std::vector<void*> bufs(n);
        for (int r = 0; r < n; ++r) bufs[r] = data[r].data();
        EXPECT(ft::run_plan_snapshot(p, FT_SUM, FT_F64, bufs.data(), count) == FT_OK);
        for (int r = 0; r < n; ++r)
          for (uint64_t i = 0; i < count; ++i) EXPECT(std::fabs(data[r][i] - want[i]) < 1e-9);
        EXPECT(ft::plan_traffic_elems(p, ft::Blocks(count, n)) == 2ull * (n - 1) * count);
      }
      ++checked;
    }
  EXPECT(checked > 150);
  EXPECT(!ft::validate_shape(7, ft::Shape{{2, 2}, 3, false}).empty());
  EXPECT(!ft::parse_topo("2,3", "", 7).ok());
}

// Device tables: every rank of every shape passes the descriptor check, the reduce-scatter half
// leaves each block complete on exactly one rank, and a table damaged in any of the ways the check
// guards against is refused.
static void device_tables() {
  for (int n = 1; n <= 24; ++n)
    for (const ft::Shape& s : ft::executable_shapes(n)) {
      ft::Plan p = ft::build_plan(n, s);
      for (int r = 0; r < n; ++r) EXPECT(ft::check_dev_plan(ft::build_dev_plan(p, r), n, r).empty());
      uint64_t owners = 0;
      for (uint64_t h : ft::rs_holders(p)) { EXPECT(h && !(h & (h - 1))); owners |= h; }
      EXPECT(n == 1 || owners == (1ull << n) - 1);
    }
  const ft::Plan p = ft::build_plan(7, ft::Shape{{2, 3}, 1, false});
  const ft::HostDevPlan good = ft::build_dev_plan(p, 2);
  EXPECT(ft::check_dev_plan(good, 7, 2).empty());
  EXPECT(!good.pulls.empty());
  auto broken = [&](auto&& damage) {
    ft::HostDevPlan d = good;
    damage(d);
    return !ft::check_dev_plan(d, 7, 2).empty();
  };
  EXPECT(broken([](ft::HostDevPlan& d) { d.pulls[0].block = 7; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.pulls[0].src[0] = 9; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.pulls[0].src[0] = 2; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.pulls[0].nsrc = 0; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.pulls[0].nsrc = FT_MAX_FANIN; d.pulls[0].reduce = 1; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.stages[0].sync_mask = 0; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.stages[0].sync_mask |= 1ull << 7; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.stages[1].pull_begin += 1; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.stages[d.plan.nstages - 1].pull_end += 1; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.nstages += 1; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.stages[0].last_rs = 1; }));
  EXPECT(broken([](ft::HostDevPlan& d) { d.plan.end_sync_mask = ~0ull; }));
  EXPECT(!ft::check_dev_plan(good, 7, 7).empty());
}

// Heap offsets: allocations alone are consecutive from zero; live blocks never overlap and stay inside the
// heap under a random mix of alloc and free; everything merges back into one block; two allocators fed the
// same sequence agree (that is what keeps the ranks' heaps symmetric).
static void heap_offsets() {
  ft::HeapAllocator h(1 << 20);
  EXPECT(h.alloc(1) == 0 && h.alloc(256) == 256 && h.alloc(257) == 512 && h.alloc(0) == 1024);
  EXPECT(h.used_bytes() == 256 + 256 + 512 + 256 && h.live_blocks() == 4);
  EXPECT(h.alloc((size_t)1 << 20) == ft::HeapAllocator::kNone);
  EXPECT(h.alloc(~(size_t)0) == ft::HeapAllocator::kNone);
  EXPECT(!h.free(128) && !h.free(4096));
  EXPECT(h.free(256) && !h.free(256));
  EXPECT(h.alloc(300) == 1280);          // the 256-byte hole is too small: first fit moves on
  EXPECT(h.alloc(200) == 256);           // and takes it for something that fits
  h.reset();
  EXPECT(h.largest_free() == (size_t)1 << 20 && h.live_blocks() == 0);

  ft::HeapAllocator a(1 << 22), b(1 << 22);
  std::vector<std::pair<size_t, size_t>> live;   // offset, requested bytes
  uint64_t rng = 12345;
  auto next = [&] { rng = rng * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(rng >> 33); };
  for (int step = 0; step < 20000; ++step) {
    if (live.empty() || next() % 3) {
      const size_t want = 1 + next() % 60000;
      const size_t off = a.alloc(want);
      EXPECT(off == b.alloc(want));
      if (off == ft::HeapAllocator::kNone) { EXPECT(a.largest_free() < ((want + 255) / 256) * 256); continue; }
      EXPECT(off % 256 == 0 && off + want <= a.size());
      for (const auto& l : live) EXPECT(off + want <= l.first || l.first + ((l.second + 255) / 256) * 256 <= off);
      live.push_back({off, want});
    } else {
      const size_t k = next() % live.size();
      EXPECT(a.free(live[k].first) && b.free(live[k].first));
      live[k] = live.back();
      live.pop_back();
    }
  }
  for (const auto& l : live) EXPECT(a.free(l.first));
  EXPECT(a.live_blocks() == 0 && a.free_blocks() == 1 && a.largest_free() == a.size());
}

// Process world: five forked children meet in a session, reduce a private buffer (pulled with
// process_vm_readv), a small one (through the segment) and one in the symmetric heap, for a lonely layout.
static void proc_world_forked() {
  {   // some sandboxes filter process_vm_readv out altogether: probe it on this process's own memory
    char src[8] = "probe", dst[8] = {0};
    struct iovec lv{dst, sizeof dst}, rv{src, sizeof src};
    if (process_vm_readv(getpid(), &lv, 1, &rv, 1, 0) != (ssize_t)sizeof src) {
      std::printf("process world not exercised: process_vm_readv is not available here\n");
      return;
    }
  }
  const int n = 5;
  const std::string session = "selftest-" + std::to_string((long)getpid());
  std::vector<pid_t> kids;
  for (int r = 0; r < n; ++r) {
    const pid_t pid = fork();
    if (pid == 0) {
      int bad = 0;
      {
        ft::ProcWorld w;
        if (!w.join(session, r, n, 30.0)) _exit(10);
        const ft::Plan p = ft::build_plan(n, ft::Shape{{2, 2}, 1, false});
        for (uint64_t count : {9ull, 70001ull}) {
          std::vector<double> v(count);
          for (int round = 0; round < 3; ++round) {
            for (uint64_t i = 0; i < count; ++i) v[i] = (double)(r + 1) + (double)(i % 5) + round;
            bad |= w.allreduce(p, FT_SUM, FT_F64, nullptr, v.data(), count).code != FT_OK;
            for (uint64_t i = 0; i < count; ++i) bad |= v[i] != 15.0 + n * ((double)(i % 5) + round);
          }
        }
        bad |= !w.heap_create(1 << 20);
        double* h = bad ? nullptr : (double*)w.heap_alloc(30000 * sizeof(double));
        if (h && w.heap_symmetric(h)) {
          for (int i = 0; i < 30000; ++i) h[i] = (double)(r + 1);
          bad |= w.allreduce(p, FT_SUM, FT_F64, nullptr, h, 30000).code != FT_OK;
          bad |= h[0] != 15.0 || h[29999] != 15.0;
        } else {
          bad = 1;
        }
        bad |= w.barrier().code != FT_OK;
      }
      _exit(bad ? 11 : 0);
    }
    kids.push_back(pid);
  }
  for (pid_t k : kids) {
    int status = 0;
    waitpid(k, &status, 0);
    EXPECT(WIFEXITED(status) && WEXITSTATUS(status) == 0);
  }
}

static void enumerators_and_models() {
  for (int n = 0; n <= 200; ++n) {
    auto a = ft::candidate_shapes(n);
    if (n >= 2) EXPECT(a.size() == ft::count_ordered_factorizations(n) + 1);
    (void)ft::candidate_shapes_legacy(n);
    (void)ft::choose_width(n);
    (void)ft::prime_factors(n);
  }
  EXPECT(ft::shape_to_string(ft::choose_v0(8).widths) == "1*8");
  EXPECT(std::fabs(ft::choose_v0(8).cost - 0.666) < 1e-9);
  ft::V1Params k;
  k.nvls_gbs = 500;
  for (int n = 2; n <= 16; ++n)
    for (uint64_t b : {1024ull, 1ull << 20, 1ull << 30}) EXPECT(std::isfinite(ft::pick_algorithm(n, b, k).us));
}

// The selection policy and its JSON reader under the sanitizers: well-formed, damaged and hostile texts, rows that
// parse but do not apply, and more distinct message sizes than the answer cache holds.
static void policy_and_json() {
  const char* texts[] = {
      "{\"params\": {\"launch_us\": 3.5, \"peer_eff\": {\"2\": 0.5, \"99\": 1.0, \"x\": 2}}, \"table\": {\"8\": [[1024, \"ll\", \"2*4\"], "
      "[1048576, \"nvls\", \"8\"], [4096, \"warp\", \"8\"], [8192, \"staged\", \"3*3\"], [1, 2], \"row\", [65536, \"hybrid-0.8-0.25\", \"8\"]]}}",
      "", "{", "{\"table\": [[[[[[[[[[", "{\"a\": \"\\u12", "{\"a\": 1e99999, \"b\": -}", "[1, 2, 3]", "nul", "{\"params\": 5, \"table\": 7}",
      "{\"table\": {\"8\": {\"not\": \"a list\"}}}"};
  int i = 0;
  for (const char* t : texts) {
    ft::Json root;
    ft::JsonParser jp(t);
    const bool ok = jp.parse(&root);
    EXPECT(ok == (i == 0 || i == 6 || i == 8 || i == 9));
    ++i;
  }
  std::string deep(5000, '[');
  ft::Json root;
  ft::JsonParser jp(deep);
  EXPECT(!jp.parse(&root));
  ft::Policy pol(8);
  EXPECT(pol.add_row(1024, "ll", "2*4") && pol.add_row(1 << 20, "nvls", "8") && pol.add_row(65536, "hybrid-0.8-0.25", "8"));
  EXPECT(!pol.add_row(4096, "warp", "8") && !pol.add_row(8192, "staged", "3*3") && !pol.add_row(8192, "staged", "2**"));
  ft::PolicyChoice c = pol.choose(1024, false, false, 64 << 20, 8 << 10);
  EXPECT(c.algo == "ll" && c.shape.widths.size() == 2 && c.from_table);
  c = pol.choose(1 << 20, true, true, 64 << 20, 8 << 10);
  EXPECT(c.algo == "nvls");
  c = pol.choose(1 << 20, true, false, 64 << 20, 8 << 10);     // the switch is not available: the row does not apply
  EXPECT(c.algo != "nvls" && c.algo != "hybrid");
  for (uint64_t b = 16; b < 16 * 3 * ft::Policy::kCacheEntries; b += 16) {   // the cache starts over instead of growing
    c = pol.choose(b, (b / 16) % 2 == 0, false, 64 << 20, 8 << 10);
    EXPECT(!c.algo.empty() && ft::validate_shape(8, c.shape).empty());
  }
  ft::Shape sh;
  EXPECT(ft::parse_shape_text(" 2 x 2 + 1 ", &sh) && sh.lonely == 1 && sh.widths.size() == 2);
  EXPECT(ft::parse_shape_text("RING8", &sh) && sh.ring);
  EXPECT(!ft::parse_shape_text("2*-4", &sh) && !ft::parse_shape_text("", &sh) && !ft::parse_shape_text("ring", &sh) &&
         !ft::parse_shape_text("99999999*2", &sh));
}

// Descriptor passing (how VMM heaps and multicast objects reach the other ranks): a pipe's read end travels from a thread
// to this one with its tag, the received descriptor reads what the sender wrote, waits run out instead of blocking.
static void fd_passing() {
  const std::string name = "ft-selftest-" + std::to_string((long)getpid());
  const int sock = ft_fd_listen(name.c_str());
  EXPECT(sock >= 0);
  int tag = -1;
  EXPECT(ft_fd_recv(sock, &tag, 50) < 0);                        // nobody sent: the wait is bounded
  EXPECT(ft_fd_send("ft-selftest-nobody-listens", 0, 1, 50) != 0);
  int pipefd[2];
  EXPECT(pipe(pipefd) == 0);
  std::thread sender([&] {
    EXPECT(write(pipefd[1], "heap", 4) == 4);
    EXPECT(ft_fd_send(name.c_str(), pipefd[0], 7, 2000) == 0);
  });
  const int got = ft_fd_recv(sock, &tag, 2000);
  sender.join();
  EXPECT(got >= 0 && tag == 7);
  char buf[8] = {0};
  EXPECT(got >= 0 && read(got, buf, 4) == 4 && !std::memcmp(buf, "heap", 4));
  if (got >= 0) ft_fd_close(got);
  ft_fd_close(pipefd[0]);
  ft_fd_close(pipefd[1]);
  ft_fd_close(sock);
}

static void thread_world(bool with_fault) {
  for (const char* text : {"2,2", "2,3", "2,2,2"}) {
    ft::ShapeConfig cfg = ft::parse_topo(text, std::string(text) == "2,3" ? "1" : "", std::string(text) == "2,2" ? 4 : (std::string(text) == "2,3" ? 7 : 8));
    EXPECT(cfg.ok());
    const int n = cfg.shape.world();
    ft::Plan p = ft::build_plan(n, cfg.shape);
    ft::CpuWorld w(n);
    w.timeout_s = with_fault ? 0.2 : 20.0;
    const uint64_t count = 4099;
    std::vector<std::vector<float>> data(n, std::vector<float>(count));
    std::vector<ft::RankStatus> st(n);
    ft::FaultSpec f;
    f.kind = ft::Fault::NeverSignal; f.rank = 1; f.stage = 1;
    for (int round = 0; round < 3; ++round) {
      for (int r = 0; r < n; ++r) for (uint64_t i = 0; i < count; ++i) data[r][i] = (float)(r + 1);
      std::vector<std::thread> th;
      for (int r = 0; r < n; ++r)
        th.emplace_back([&, r] { st[r] = ft::cpu_allreduce(w, r, p, FT_SUM, FT_F32, nullptr, data[r].data(), count, 0, with_fault ? &f : nullptr); });
      for (auto& t : th) t.join();
      if (with_fault) {
        bool any_timeout = false;
        for (int r = 0; r < n; ++r) any_timeout = any_timeout || st[r].code == FT_ERR_TIMEOUT;
        EXPECT(any_timeout);
        break;   // the world is poisoned after a fault
      }
      for (int r = 0; r < n; ++r) { EXPECT(st[r].code == FT_OK); EXPECT(data[r][count - 1] == (float)(n * (n + 1) / 2)); }
    }
  }
}

// Reduce-scatter and all-gather as calls of their own, three rounds without any host barrier in
// between, with a whole all-reduce after each pair: rendezvous numbers keep growing across the three
// kinds of call and the closing all-rank rendezvous lets every rank overwrite its buffer right away.
static void thread_world_phases() {
  for (const char* text : {"2,2", "2,3", "2,2,2", "1"}) {
    const std::string t = text;
    const int n = t == "2,2" ? 4 : (t == "2,3" ? 7 : (t == "1" ? 5 : 8));
    ft::ShapeConfig cfg = ft::parse_topo(text, t == "2,3" ? "1" : "", n);
    EXPECT(cfg.ok());
    ft::Plan p = ft::build_plan(n, cfg.shape);
    const std::vector<uint64_t> holders = ft::rs_holders(p);
    ft::CpuWorld w(n);
    w.timeout_s = 20.0;
    const uint64_t count = 1031;
    const ft::Blocks g(count, n);
    std::vector<std::vector<double>> data(n, std::vector<double>(count));
    std::vector<int> bad(n, 0);
    std::vector<std::thread> th;
    for (int r = 0; r < n; ++r)
      th.emplace_back([&, r] {
        for (int round = 0; round < 3; ++round) {
          for (uint64_t i = 0; i < count; ++i) data[r][i] = (double)(r + 1 + round);
          bad[r] |= ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, data[r].data(), count, 0, nullptr, 1, 1).code != FT_OK;
          for (int b = 0; b < n; ++b)   // wipe everything this rank does not own
            if (!(holders[b] >> r & 1))
              for (uint64_t i = g.offset(b); i < g.offset(b) + g.length(b); ++i) data[r][i] = -1e300;
          bad[r] |= ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, data[r].data(), count, 0, nullptr, 1, 2).code != FT_OK;
          bad[r] |= ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, data[r].data(), count).code != FT_OK;
          const double want = (double)n * (n * (n + 1) / 2 + n * round);
          for (uint64_t i = 0; i < count; ++i) bad[r] |= data[r][i] != want;
        }
      });
    for (auto& x : th) x.join();
    for (int r = 0; r < n; ++r) EXPECT(!bad[r]);
  }
}

// Host twins of the small-message protocols, mixed with staged calls and single phases, with every rank
// delayed at random before each call.  Neither protocol closes with a rendezvous; what keeps a slow rank's
// reads apart from a fast rank's next write into the same slot (two calls later) is only the argument
// that finishing the call in between needs every rank's contribution.  Under the thread sanitizer a hole
// in that argument is a reported race; in any build it is a wrong sum or a timeout.
static void random_pause(int rank) {
  thread_local uint64_t rng = 0;
  if (!rng) rng = 7777 + 13 * (uint64_t)rank;
  rng = rng * 6364136223846793005ull + 1442695040888963407ull;
  if ((rng >> 60) < 5) std::this_thread::sleep_for(std::chrono::microseconds((rng >> 40) % 400));
}

// Every executable shape up to 9 ranks on real threads that stall at random between a stage's rendezvous and
// its pulls, six calls back to back: in place, through the slots, and as two single phases.  The per-stage rendezvous sets are the
// only thing that orders one rank's writes against another's reads; a set that misses a dependency shows up
// as a race under the thread sanitizer (and usually as a wrong sum).
static void thread_world_all_shapes() {
  int shapes = 0;
  for (int n = 2; n <= 9; ++n)
    for (const ft::Shape& s : ft::executable_shapes(n)) {
      const ft::Plan p = ft::build_plan(n, s);
      ft::CpuWorld w(n);
      w.timeout_s = 30.0;
      w.mid_call_hook = random_pause;
      const uint64_t count = 97;
      const std::vector<uint64_t> holders = ft::rs_holders(p);
      const ft::Blocks g(count, n);
      std::vector<int> bad(n, 0);
      std::vector<std::thread> th;
      for (int r = 0; r < n; ++r)
        th.emplace_back([&, r] {
          std::vector<double> buf(count);
          for (int round = 0; round < 6; ++round) {
            for (uint64_t i = 0; i < count; ++i) buf[i] = (double)(r + 1) * (double)(i + 1) + round;
            ft::RankStatus st;
            if (round % 3 == 0) {
              st = ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, buf.data(), count);
            } else if (round % 3 == 1) {
              st = ft::cpu_allreduce_slots(w, r, p, FT_SUM, FT_F64, nullptr, buf.data(), count);
            } else {   // the two halves as calls of their own, everything not owned wiped in between
              st = ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, buf.data(), count, 0, nullptr, 1, 1);
              for (int b = 0; b < n; ++b)
                if (!(holders[b] >> r & 1))
                  for (uint64_t i = g.offset(b); i < g.offset(b) + g.length(b); ++i) buf[i] = -1e300;
              if (st.code == FT_OK) st = ft::cpu_allreduce(w, r, p, FT_SUM, FT_F64, nullptr, buf.data(), count, 0, nullptr, 1, 2);
            }
            bad[r] |= st.code != FT_OK;
            for (uint64_t i = 0; i < count; ++i) bad[r] |= buf[i] != (double)(n * (n + 1) / 2) * (double)(i + 1) + (double)n * round;
          }
        });
      for (auto& x : th) x.join();
      for (int r = 0; r < n; ++r) EXPECT(!bad[r]);
      ++shapes;
    }
  EXPECT(shapes > 30);
}

static void thread_world_small_message_twins() {
  for (int n : {2, 3, 5, 8}) {
    ft::CpuWorld w(n);
    w.timeout_s = 30.0;
    w.mid_call_hook = random_pause;   // ranks also stall in the middle of a call, between publishing and reading
    const ft::Plan flat = ft::build_plan(n, ft::Shape::flat(n));
    const ft::Plan ring = ft::build_plan(n, ft::Shape::make_ring(n));
    const ft::Plan tree = ft::build_plan(n, n == 8 ? ft::Shape{{2, 4}, 0, false} : (n == 5 ? ft::Shape{{2, 2}, 1, false} : ft::Shape::flat(n)));
    const uint64_t count = 777;
    std::vector<int> bad(n, 0);
    std::vector<std::thread> th;
    for (int r = 0; r < n; ++r)
      th.emplace_back([&, r] {
        uint64_t rng = 99 + r;
        auto jitter = [&] {
          rng = rng * 6364136223846793005ull + 1442695040888963407ull;
          std::this_thread::sleep_for(std::chrono::microseconds((rng >> 40) % 300));
        };
        std::vector<float> buf(count);
        for (int round = 0; round < 120; ++round) {
          for (uint64_t i = 0; i < count; ++i) buf[i] = (float)(r + 1) + (float)(i % 7) + (float)round;
          jitter();
          ft::RankStatus st;
          switch (round % 10) {   // back-to-back calls of the same kind are the ones that lean on the parity rule
            case 0: case 1: case 6: st = ft::cpu_allreduce_ll(w, r, FT_SUM, FT_F32, nullptr, buf.data(), count); break;
            case 2: case 3: case 5: st = ft::cpu_allreduce_oneshot(w, r, FT_SUM, FT_F32, nullptr, buf.data(), count); break;
            case 4: st = ft::cpu_allreduce(w, r, round % 16 == 4 ? flat : ring, FT_SUM, FT_F32, nullptr, buf.data(), count); break;
            case 9: st = ft::cpu_allreduce_push(w, r, FT_SUM, FT_F32, buf.data(), count); break;
            case 8:   // a plan on tagged words, twice in a row (both receive areas), then the flat tagged-word call on the same areas
              st = ft::cpu_allreduce_ll_tree(w, r, round % 20 == 8 ? tree : ring, FT_SUM, FT_F32, nullptr, buf.data(), count);
              if (st.code == FT_OK) {
                for (uint64_t i = 0; i < count; ++i) buf[i] = (float)(r + 1) + (float)(i % 7) + (float)round;
                st = ft::cpu_allreduce_ll_tree(w, r, flat, FT_SUM, FT_F32, nullptr, buf.data(), count);
              }
              break;
            case 7:   // through the slots, twice in a row, with different shapes (no closing rendezvous in this mode)
              st = ft::cpu_allreduce_slots(w, r, round % 16 == 7 ? tree : ring, FT_SUM, FT_F32, nullptr, buf.data(), count);
              if (st.code == FT_OK) {
                for (uint64_t i = 0; i < count; ++i) buf[i] = (float)(r + 1) + (float)(i % 7) + (float)round;
                st = ft::cpu_allreduce_slots(w, r, flat, FT_SUM, FT_F32, nullptr, buf.data(), count);
              }
              break;
            default:
              st = ft::cpu_allreduce(w, r, flat, FT_SUM, FT_F32, nullptr, buf.data(), count, 0, nullptr, 1, 1);
              if (st.code == FT_OK) st = ft::cpu_allreduce(w, r, flat, FT_SUM, FT_F32, nullptr, buf.data(), count, 0, nullptr, 1, 2);
          }
          bad[r] |= st.code != FT_OK;
          for (uint64_t i = 0; i < count; ++i) {
            const float want = (float)(n * (n + 1) / 2) + (float)n * ((float)(i % 7) + (float)round);
            bad[r] |= buf[i] != want;
          }
        }
      });
    for (auto& x : th) x.join();
    for (int r = 0; r < n; ++r) EXPECT(!bad[r]);
  }
}

int main(int argc, char** argv) {
  const bool threads = argc > 1 && !std::strcmp(argv[1], "threads");
  if (!threads) { proc_world_forked(); plans_and_snapshot(); device_tables(); heap_offsets(); enumerators_and_models(); policy_and_json(); fd_passing(); }
  thread_world(false);
  thread_world_phases();
  thread_world_small_message_twins();
  thread_world_all_shapes();
  thread_world(true);
  std::printf(fails ? "%d FAILURES\n" : "selftest ok\n", fails);
  return fails ? 1 : 0;
}
