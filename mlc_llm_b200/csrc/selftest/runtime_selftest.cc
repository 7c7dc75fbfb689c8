// Stand-alone exerciser of the native serving runtime, built with -fsanitize=address,undefined or
// -fsanitize=thread by tests/test_sanitizers_cpu.py (no Python, no GPU): the paged KV manager, the radix
// tree and prefix cache under random operation sequences, and a full engine with a deterministic
// in-process model backend driven through the threaded engine by several client threads that add and
// abort requests while the two background loops run.
//
// The reference keeps its runtime memory- and race-clean with the sanitizer builds of its CI; this
// program is the counterpart for this runtime's C++ (csrc/serve/*.cc except the Python bindings).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <random>
#include <set>
#include <thread>

#include "config.h"
#include "engine.h"
#include "kv_manager.h"
#include "prefix_cache.h"
#include "radix_tree.h"
#include "tokenizer.h"

using namespace mlcb;

#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::fprintf(stderr, "CHECK failed at %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      std::exit(1);                                                              \
    }                                                                            \
  } while (0)

namespace {

constexpr int kVocab = 512;

// ------------------------------------------------------------------ paged KV manager
void TestKVManager(uint64_t seed) {
  std::mt19937_64 rng(seed);
  KVManager kv(256, 16, 32);
  std::map<int64_t, int64_t> len;  // model of the sequence lengths
  int64_t next_id = 0;
  for (int step = 0; step < 600; ++step) {
    const int op = static_cast<int>(rng() % 6);
    if (op == 0 || len.empty()) {
      if (len.size() >= 24) continue;
      kv.AddSequence(next_id);
      if (rng() % 4 == 0) kv.EnableSlidingWindow(next_id, 48, 4);
      len[next_id++] = 0;
    } else if (op <= 2) {
      // append to a few sequences at once
      std::vector<int64_t> ids;
      std::vector<int32_t> lens;
      int64_t need = 0;
      for (auto& kvp : len) {
        if (rng() % 3) continue;
        const int32_t n = 1 + static_cast<int32_t>(rng() % 40);
        need += kv.PagesNeeded(kvp.first, n);
        ids.push_back(kvp.first);
        lens.push_back(n);
      }
      if (ids.empty() || need > kv.NumAvailablePages()) continue;
      ForwardPlan plan = kv.BeginForward(ids, lens);
      size_t total = 0;
      for (size_t i = 0; i < ids.size(); ++i) {
        len[ids[i]] += lens[i];
        total += static_cast<size_t>(lens[i]);
        CHECK(kv.SequenceLength(ids[i]) == len[ids[i]]);
      }
      CHECK(plan.slots.size() == total && plan.positions.size() == total);
      CHECK(plan.page_indptr.size() == ids.size() + 1);
      // the copies of one plan run in one launch: no pair writes what another reads or writes
      {
        std::set<int32_t> srcs, dsts;
        for (size_t i = 0; i + 1 < plan.page_copies.size(); i += 2) {
          srcs.insert(plan.page_copies[i]);
          CHECK(dsts.insert(plan.page_copies[i + 1]).second);
        }
        for (int32_t d : dsts) CHECK(!srcs.count(d));
      }
      if (rng() % 5 == 0) {
        // a plan whose forward does not run after all: its rows are popped, its copies ride on the next plan
        for (size_t i = 0; i < ids.size(); ++i) {
          kv.PopN(ids[i], lens[i]);
          len[ids[i]] -= lens[i];
        }
        kv.RequeuePlanSideEffects(plan);
        std::vector<int32_t> ones(ids.size(), 1);
        int64_t again = 0;
        for (int64_t id : ids) again += kv.PagesNeeded(id, 1);
        if (again <= kv.NumAvailablePages()) {
          ForwardPlan next = kv.BeginForward(ids, ones);
          for (int64_t id : ids) len[id] += 1;
          for (size_t i = 0; i + 1 < plan.page_copies.size(); i += 2) {
            bool found = false;
            for (size_t j = 0; j + 1 < next.page_copies.size(); j += 2)
              found |= next.page_copies[j + 1] == plan.page_copies[i + 1];
            CHECK(found);  // every destination that is still owned gets its copy
          }
        }
      }
      // no two appended tokens share a slot
      std::set<int32_t> seen(plan.slots.begin(), plan.slots.end());
      CHECK(seen.size() == total);
    } else if (op == 3) {
      auto it = len.begin();
      std::advance(it, rng() % len.size());
      if (it->second == 0 || len.size() >= 24 || kv.NumAvailablePages() < 2) continue;
      const int64_t at = static_cast<int64_t>(rng() % static_cast<uint64_t>(it->second + 1));
      try {
        kv.ForkSequence(it->first, next_id, at);
      } catch (const std::exception&) {
        continue;  // a windowed sequence that has released pages cannot be forked
      }
      len[next_id] = at;
      CHECK(kv.SequenceLength(next_id) == at);
      ++next_id;
    } else if (op == 4) {
      auto it = len.begin();
      std::advance(it, rng() % len.size());
      if (it->second == 0) continue;
      const int64_t n = 1 + static_cast<int64_t>(rng() % static_cast<uint64_t>(std::min<int64_t>(it->second, 8)));
      try {
        kv.PopN(it->first, n);
        it->second -= n;
      } catch (const std::exception&) {
        // a windowed sequence refuses to go back behind what it has released
      }
    } else {
      auto it = len.begin();
      std::advance(it, rng() % len.size());
      kv.RemoveSequence(it->first);
      len.erase(it);
    }
  }
  for (auto& kvp : len) kv.RemoveSequence(kvp.first);
  CHECK(kv.NumSequences() == 0);
  CHECK(kv.NumAvailablePages() == kv.NumPages());
}

// ------------------------------------------------------------------ radix tree + prefix cache
void TestRadixTree(uint64_t seed) {
  std::mt19937_64 rng(seed);
  RadixTree tree(1 << 12);
  const int64_t capacity = tree.FreeCapacity();
  std::map<int64_t, std::vector<int32_t>> model;
  int64_t next_id = 0;
  for (int step = 0; step < 800; ++step) {
    const int op = static_cast<int>(rng() % 7);
    if (op == 0 || model.empty()) {
      tree.Add(next_id);
      model[next_id++] = {};
      continue;
    }
    auto it = model.begin();
    std::advance(it, rng() % model.size());
    if (op <= 2) {
      std::vector<int32_t> toks(1 + rng() % 70);
      for (auto& t : toks) t = 1 + static_cast<int32_t>(rng() % 3);
      tree.Extend(it->first, toks);
      it->second.insert(it->second.end(), toks.begin(), toks.end());
    } else if (op == 3) {
      const int64_t at = static_cast<int64_t>(rng() % (it->second.size() + 1));
      tree.Fork(next_id, it->first, at);
      model[next_id++] = std::vector<int32_t>(it->second.begin(), it->second.begin() + at);
    } else if (op == 4 && !it->second.empty()) {
      const int64_t n = 1 + static_cast<int64_t>(rng() % it->second.size());
      tree.Rollback(it->first, n);
      it->second.resize(it->second.size() - static_cast<size_t>(n));
    } else if (op == 5) {
      tree.Remove(it->first);
      model.erase(it);
    } else {
      std::vector<int32_t> q(it->second.begin(), it->second.begin() + static_cast<long>(rng() % (it->second.size() + 1)));
      q.push_back(9);
      auto m = tree.Match(q);
      CHECK(m.first >= static_cast<int64_t>(q.size()) - 1);
    }
    if (step % 50 == 0)
      for (auto& kvp : model) CHECK(tree.Get(kvp.first) == kvp.second);
  }
  for (auto& kvp : model) tree.Remove(kvp.first);
  CHECK(tree.FreeCapacity() == capacity);

  // prefix cache: insert / extend / recycle / reuse, eviction through the callback
  std::vector<int64_t> removed;
  PrefixCache pc(true, 4, [&](int64_t id) { removed.push_back(id); });
  std::vector<int64_t> live;
  for (int64_t id = 0; id < 60; ++id) {
    std::vector<int32_t> toks(20 + rng() % 100);
    for (auto& t : toks) t = 1 + static_cast<int32_t>(rng() % 2);
    PrefixMatch m = pc.InsertSequence(id, toks);
    CHECK(m.prefilled_offset <= static_cast<int64_t>(toks.size()));
    // a recycled sequence that is taken over keeps its own id
    const int64_t owner = m.reused_seq_id >= 0 ? m.reused_seq_id : id;
    CHECK(pc.HasSequence(owner));
    pc.ExtendSequence(owner, std::vector<int32_t>(toks.begin() + m.prefilled_offset, toks.end()));
    pc.CommitSequenceExtention();
    CHECK(pc.SequenceLength(owner) == static_cast<int64_t>(toks.size()));
    live.push_back(owner);
    if (live.size() > 2) {
      pc.RecycleSequence(live.front(), (rng() % 2) != 0);
      live.erase(live.begin());
    }
  }
  CHECK(!removed.empty());
  CHECK(pc.NumRecycling() <= 4);
}

}  // namespace

namespace {

// ------------------------------------------------------------------ engine behind the threaded engine
// Deterministic stand-in for the model: the token sampled for a row depends only on the position and
// the token that was fed there, so every request's output can be predicted by the client.
class FakeBackend : public ModelBackend {
 public:
  static int32_t Next(int32_t token, int32_t position) { return 3 + (token * 31 + position * 7) % (kVocab - 3); }

  SampleOutput ForwardSample(int, const ForwardPlan& plan, const std::vector<int32_t>& token_ids,
                             const std::vector<int64_t>&, const SampleParams& sampling) override {
    calls_.fetch_add(1);
    SampleOutput out;
    for (int32_t row : sampling.logit_token_index) {
      out.tokens.push_back(Next(token_ids[static_cast<size_t>(row)], plan.positions[static_cast<size_t>(row)]));
      out.probs.push_back(1.f);
    }
    return out;
  }
  VerifyOutput ForwardVerify(int, const ForwardPlan&, const std::vector<int32_t>&, const VerifyParams&) override {
    throw std::runtime_error("the self-test runs without speculative decoding");
  }
  void MoveKVTokens(int, const std::vector<int32_t>&) override {}
  int64_t calls() const { return calls_.load(); }

 private:
  std::atomic<int64_t> calls_{0};
};

std::shared_ptr<Tokenizer> MakeTokenizer() {
  std::vector<std::string> vocab;
  for (int i = 0; i < kVocab; ++i) vocab.push_back("t" + std::to_string(i) + "_");
  TokenizerInfo info;
  info.token_postproc_method = "byte_level";
  return std::make_shared<Tokenizer>(vocab, info, [](const std::string& s) {
    std::vector<int32_t> ids;
    for (unsigned char c : s) ids.push_back(3 + c % (kVocab - 3));
    return ids;
  });
}

void TestThreadedEngine(uint64_t seed) {
  auto tokenizer = MakeTokenizer();
  auto backend = std::make_shared<FakeBackend>();
  std::mutex mu;
  std::map<std::string, std::vector<int32_t>> got;
  std::map<std::string, std::string> finished;
  ThreadedEngine::EngineFactory factory = [&](const std::string& cfg_json, StreamCallback cb) {
    EngineModelInfo info;
    info.vocab_size = kVocab;
    info.num_pages = 512;
    info.eos_token_ids = {2};
    info.generation_defaults_json = "{\"temperature\": 0.0, \"top_p\": 1.0}";
    return Engine::Create(EngineConfig::FromJSON(cfg_json), {info}, backend, tokenizer, nullptr, nullptr,
                          std::move(cb));
  };
  ThreadedEngine engine(factory, [&](std::vector<RequestStreamOutput> outs) {
    std::lock_guard<std::mutex> lock(mu);
    for (auto& o : outs) {
      if (!o.group_delta_token_ids.empty())
        got[o.request_id].insert(got[o.request_id].end(), o.group_delta_token_ids[0].begin(),
                                 o.group_delta_token_ids[0].end());
      if (!o.group_finish_reason.empty() && !o.group_finish_reason[0].empty())
        finished[o.request_id] = o.group_finish_reason[0];
    }
  });
  std::thread loop([&] { engine.RunBackgroundLoop(); });
  std::thread stream([&] { engine.RunBackgroundStreamBackLoop(); });
  engine.Reload(
      "{\"mode\": \"server\", \"max_num_sequence\": 16, \"max_total_sequence_length\": 4096, "
      "\"max_single_sequence_length\": 1024, \"prefill_chunk_size\": 64, \"kv_cache_page_size\": 16, "
      "\"prefix_cache_mode\": \"radix\", \"prefix_cache_max_num_recycling_seqs\": 8}");
  const GenerationConfig defaults = engine.DefaultGenerationConfig();

  constexpr int kClients = 4, kPerClient = 24;
  std::map<std::string, std::pair<std::vector<int32_t>, int>> sent;  // id -> (prompt, max_tokens)
  std::set<std::string> aborted;
  std::mutex sent_mu;
  std::vector<std::thread> clients;
  for (int c = 0; c < kClients; ++c) {
    clients.emplace_back([&, c] {
      std::mt19937_64 rng(seed * 977 + static_cast<uint64_t>(c));
      for (int i = 0; i < kPerClient; ++i) {
        Request r;
        r.id = "c" + std::to_string(c) + "-" + std::to_string(i);
        InputItem item;
        // many prompts share a prefix so the prefix cache forks and reuses sequences
        const int shared = static_cast<int>(rng() % 3) * 20;
        for (int k = 0; k < shared; ++k) item.tokens.push_back(5 + k % 7);
        const int own = 1 + static_cast<int>(rng() % 90);
        for (int k = 0; k < own; ++k) item.tokens.push_back(3 + static_cast<int32_t>(rng() % (kVocab - 3)));
        const int max_tokens = 1 + static_cast<int>(rng() % 24);
        r.prompt_tokens = static_cast<int64_t>(item.tokens.size());
        r.cfg = GenerationConfig::FromJSON(
            "{\"max_tokens\": " + std::to_string(max_tokens) + ", \"temperature\": 0.0, \"debug_config\": {\"ignore_eos\": true}}",
            defaults);
        {
          std::lock_guard<std::mutex> lock(sent_mu);
          sent[r.id] = {item.tokens, max_tokens};
        }
        r.inputs.push_back(std::move(item));
        const std::string id = r.id;
        engine.AddRequest(std::move(r));
        if (rng() % 6 == 0) {
          std::this_thread::sleep_for(std::chrono::microseconds(rng() % 400));
          {
            std::lock_guard<std::mutex> lock(sent_mu);
            aborted.insert(id);
          }
          engine.AbortRequest(id);
        }
        if (rng() % 3 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 300));
      }
    });
  }
  for (auto& t : clients) t.join();
  // wait until every request that was not aborted has finished
  for (int spin = 0; spin < 20000; ++spin) {
    {
      std::lock_guard<std::mutex> lock(mu);
      size_t done = 0;
      for (auto& kvp : sent) done += (finished.count(kvp.first) || aborted.count(kvp.first)) ? 1 : 0;
      if (done == sent.size()) break;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  const std::string metrics = engine.JSONMetrics();
  CHECK(!metrics.empty());
  engine.Reset();
  engine.Unload();
  engine.ExitBackgroundLoop();
  loop.join();
  stream.join();

  std::lock_guard<std::mutex> lock(mu);
  int checked = 0;
  for (auto& kvp : sent) {
    if (aborted.count(kvp.first)) continue;
    CHECK(finished.count(kvp.first));
    CHECK(finished[kvp.first] == "length");
    // replay the deterministic model
    const auto& prompt = kvp.second.first;
    std::vector<int32_t> want;
    int32_t tok = prompt.back();
    int32_t pos = static_cast<int32_t>(prompt.size()) - 1;
    for (int k = 0; k < kvp.second.second; ++k) {
      tok = FakeBackend::Next(tok, pos);
      want.push_back(tok);
      ++pos;
    }
    CHECK(got[kvp.first] == want);
    ++checked;
  }
  CHECK(checked > kClients * kPerClient / 2);
  CHECK(backend->calls() > 0);
  std::printf("engine: %d requests checked, %zu aborted, %lld backend calls\n", checked, aborted.size(),
              static_cast<long long>(backend->calls()));
}

}  // namespace

int main(int argc, char** argv) {
  const uint64_t seed = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 1;
  for (uint64_t s = 0; s < 4; ++s) {
    TestKVManager(seed + s);
    TestRadixTree(seed + s);
  }
  std::printf("kv manager, radix tree, prefix cache: ok\n");
  TestThreadedEngine(seed);
  std::printf("selftest ok\n");
  return 0;
}
