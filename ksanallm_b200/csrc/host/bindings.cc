// pybind11 surface of the native host runtime: KV block manager, continuous-batching scheduler,
// step-plan packer, draft trie, load balancer. The reference exposes its engine through one
// pybind module as well (src/ksana_llm/torch_op/serving_op.cpp:84-251); here the boundary sits
// lower (scheduler / cache primitives) because each GPU rank is its own Python process.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "draft_trie.h"
#include "kv_cache.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace ksana;

static py::array_t<int32_t> PairsToArray(const std::vector<CopyPair>& v) {
  py::array_t<int32_t> a({static_cast<py::ssize_t>(v.size()), static_cast<py::ssize_t>(2)});
  auto m = a.mutable_unchecked<2>();
  for (size_t i = 0; i < v.size(); ++i) {
    m(i, 0) = v[i].src;
    m(i, 1) = v[i].dst;
  }
  return a;
}

PYBIND11_MODULE(_ksana_host, m) {
  m.doc() = "ksanallm_b200 native host runtime";

  py::class_<CacheStats>(m, "CacheStats")
      .def_readonly("prefix_query_tokens", &CacheStats::prefix_query_tokens)
      .def_readonly("prefix_hit_tokens", &CacheStats::prefix_hit_tokens)
      .def_readonly("flexible_hit_tokens", &CacheStats::flexible_hit_tokens)
      .def_readonly("evicted_blocks", &CacheStats::evicted_blocks)
      .def_readonly("merged_blocks", &CacheStats::merged_blocks)
      .def_readonly("swapped_out_blocks", &CacheStats::swapped_out_blocks)
      .def_readonly("swapped_in_blocks", &CacheStats::swapped_in_blocks);

  py::class_<KVCacheManager, std::shared_ptr<KVCacheManager>>(m, "KVCacheManager")
      .def(py::init<int, int, int, bool>(), py::arg("num_device_blocks"), py::arg("num_host_blocks"),
           py::arg("block_size"), py::arg("enable_prefix"))
      .def_property_readonly("block_size", &KVCacheManager::block_size)
      .def_property_readonly("num_device_blocks", &KVCacheManager::num_device_blocks)
      .def_property_readonly("num_host_blocks", &KVCacheManager::num_host_blocks)
      .def_property_readonly("num_free_host_blocks", &KVCacheManager::num_free_host_blocks)
      .def_property_readonly("num_available_blocks", &KVCacheManager::num_available_blocks)
      .def_property_readonly("num_free_blocks", &KVCacheManager::num_free_blocks)
      .def_property_readonly("num_cached_blocks", &KVCacheManager::num_cached_blocks)
      .def_property_readonly("stats", &KVCacheManager::stats)
      .def("has", &KVCacheManager::Has)
      .def("match_prefix", &KVCacheManager::MatchPrefix)
      .def("create_seq", &KVCacheManager::CreateSeq, py::arg("seq"), py::arg("tokens"), py::arg("use_prefix") = true)
      .def("ensure_capacity", &KVCacheManager::EnsureCapacity)
      .def("commit_filled",
           [](KVCacheManager& c, int64_t seq, const std::vector<int32_t>& tokens, int n) {
             return PairsToArray(c.CommitFilled(seq, tokens, n));
           })
      .def("block_table", &KVCacheManager::BlockTable)
      .def("flexible_reserve",
           [](KVCacheManager& c, int64_t seq, const std::vector<int32_t>& tokens, int shared, int min_len) -> py::object {
             FlexibleRun run;
             if (!c.FlexibleReserve(seq, tokens, shared, min_len, &run)) return py::none();
             return py::make_tuple(run.dst_begin, run.src_slots, run.dst_slots, run.src_pos);
           })
      .def("num_blocks", &KVCacheManager::NumBlocks)
      .def("free_seq", &KVCacheManager::FreeSeq)
      .def("truncate", &KVCacheManager::Truncate)
      .def("fork",
           [](KVCacheManager& c, int64_t parent, int64_t child) {
             std::vector<CopyPair> cp;
             bool ok = c.Fork(parent, child, &cp);
             return py::make_tuple(ok, PairsToArray(cp));
           })
      .def("swap_out",
           [](KVCacheManager& c, int64_t seq) {
             std::vector<CopyPair> cp;
             bool ok = c.SwapOut(seq, &cp);
             return py::make_tuple(ok, PairsToArray(cp));
           })
      .def("swap_in",
           [](KVCacheManager& c, int64_t seq) {
             std::vector<CopyPair> cp;
             bool ok = c.SwapIn(seq, &cp);
             return py::make_tuple(ok, PairsToArray(cp));
           })
      .def("clear_unreferenced", &KVCacheManager::ClearUnreferenced);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("block_size", &SchedulerConfig::block_size)
      .def_readwrite("max_batch_size", &SchedulerConfig::max_batch_size)
      .def_readwrite("max_step_tokens", &SchedulerConfig::max_step_tokens)
      .def_readwrite("max_token_len", &SchedulerConfig::max_token_len)
      .def_readwrite("max_waiting_queue_len", &SchedulerConfig::max_waiting_queue_len)
      .def_readwrite("waiting_timeout_ms", &SchedulerConfig::waiting_timeout_ms)
      .def_readwrite("split_fuse_token_num", &SchedulerConfig::split_fuse_token_num)
      .def_readwrite("preempt_mode", &SchedulerConfig::preempt_mode)
      .def_readwrite("launch_block_threshold", &SchedulerConfig::launch_block_threshold)
      .def_readwrite("swapin_block_threshold", &SchedulerConfig::swapin_block_threshold)
      .def_readwrite("max_draft_tokens", &SchedulerConfig::max_draft_tokens)
      .def_readwrite("ptp_mode", &SchedulerConfig::ptp_mode)
      .def_readwrite("min_flexible_cache_num", &SchedulerConfig::min_flexible_cache_num)
      .def_readwrite("pp_wb_strategy", &SchedulerConfig::pp_wb_strategy)
      .def_readwrite("lookahead_slots", &SchedulerConfig::lookahead_slots)
      .def_readwrite("decode_token_threshold", &SchedulerConfig::decode_token_threshold);

  py::class_<SchedStats>(m, "SchedStats")
      .def_readonly("steps", &SchedStats::steps)
      .def_readonly("preempt_recompute", &SchedStats::preempt_recompute)
      .def_readonly("preempt_swap", &SchedStats::preempt_swap)
      .def_readonly("swap_in", &SchedStats::swap_in)
      .def_readonly("draft_proposed", &SchedStats::draft_proposed)
      .def_readonly("mb_migrations", &SchedStats::mb_migrations)
      .def_readonly("draft_accepted", &SchedStats::draft_accepted)
      .def_readonly("timeouts", &SchedStats::timeouts)
      .def_readonly("finished", &SchedStats::finished);

  py::class_<StepEntry>(m, "StepEntry")
      .def_readonly("seq_id", &StepEntry::seq_id)
      .def_readonly("q_start", &StepEntry::q_start)
      .def_readonly("q_len", &StepEntry::q_len)
      .def_readonly("n_drafts", &StepEntry::n_drafts)
      .def_readonly("num_logits", &StepEntry::num_logits)
      .def_readonly("is_decode", &StepEntry::is_decode);

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("entries", &StepPlan::entries)
      .def_property_readonly("swap_out", [](const StepPlan& p) { return PairsToArray(p.swap_out); })
      .def_property_readonly("swap_in", [](const StepPlan& p) { return PairsToArray(p.swap_in); })
      .def_property_readonly("block_copies", [](const StepPlan& p) { return PairsToArray(p.block_copies); })
      .def_property_readonly("flexible",
                             [](const StepPlan& p) {
                               py::array_t<int32_t> a({static_cast<py::ssize_t>(p.flexible.size() / 4), py::ssize_t(4)});
                               std::copy(p.flexible.begin(), p.flexible.end(), a.mutable_data());
                               return a;
                             })
      .def_property_readonly("dropped",
                             [](const StepPlan& p) {
                               std::vector<std::pair<int64_t, int>> v;
                               for (auto& e : p.dropped) v.emplace_back(e.seq_id, e.finish_reason);
                               return v;
                             })
      .def_property_readonly("seq_ids",
                             [](const StepPlan& p) {
                               std::vector<int64_t> v;
                               for (auto& e : p.entries) v.push_back(e.seq_id);
                               return v;
                             })
      .def_readonly("num_prefill", &StepPlan::num_prefill)
      .def_readonly("num_decode", &StepPlan::num_decode)
      .def_readonly("total_tokens", &StepPlan::total_tokens)
      .def_readonly("total_logits", &StepPlan::total_logits)
      .def_readonly("max_q_len", &StepPlan::max_q_len)
      .def_readonly("max_kv_len", &StepPlan::max_kv_len)
      .def("empty", &StepPlan::empty);

  py::class_<StepResult>(m, "StepResult")
      .def_readonly("seq_id", &StepResult::seq_id)
      .def_readonly("new_tokens", &StepResult::new_tokens)
      .def_readonly("accepted_drafts", &StepResult::accepted_drafts)
      .def_readonly("finish_reason", &StepResult::finish_reason);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerConfig&, std::shared_ptr<KVCacheManager>>())
      .def_property_readonly("stats", &Scheduler::stats)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def_property_readonly("num_swapped", &Scheduler::num_swapped)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def("workload", &Scheduler::Workload)
      .def(
          "enqueue",
          [](Scheduler& s, int64_t id, const std::vector<int32_t>& tokens, int max_new_tokens, bool ignore_eos,
             const std::vector<int32_t>& eos_ids, const std::vector<int32_t>& stop_ids, int64_t arrival_ms,
             int64_t group_id, bool no_cache) {
            Sequence q;
            q.no_cache = no_cache;
            q.id = id;
            q.group_id = group_id;
            q.tokens = tokens;
            q.max_new_tokens = max_new_tokens;
            q.ignore_eos = ignore_eos;
            q.eos_ids = eos_ids;
            q.stop_ids = stop_ids;
            q.arrival_ms = arrival_ms;
            return s.Enqueue(std::move(q));
          },
          py::arg("seq_id"), py::arg("tokens"), py::arg("max_new_tokens"), py::arg("ignore_eos") = false,
          py::arg("eos_ids") = std::vector<int32_t>{}, py::arg("stop_ids") = std::vector<int32_t>{},
          py::arg("arrival_ms") = 0, py::arg("group_id") = 0, py::arg("no_cache") = false)
      .def("abort", &Scheduler::Abort)
      .def("fork", &Scheduler::Fork)
      .def("finish", &Scheduler::Finish)
      .def("replace_last_token", &Scheduler::ReplaceLastToken)
      .def("set_drafts", &Scheduler::SetDrafts)
      .def("forget", &Scheduler::Forget)
      .def("tokens",
           [](const Scheduler& s, int64_t id) {
             const Sequence* q = s.Get(id);
             return q ? q->tokens : std::vector<int32_t>{};
           })
      .def("seq_info",
           [](const Scheduler& s, int64_t id) -> py::object {
             const Sequence* q = s.Get(id);
             if (!q) return py::none();
             py::dict d;
             d["state"] = q->state;
             d["prompt_len"] = q->prompt_len;
             d["num_tokens"] = static_cast<int>(q->tokens.size());
             d["num_computed"] = q->num_computed;
             d["finish_reason"] = q->finish_reason;
             d["preempt_count"] = q->preempt_count;
             return d;
           })
      .def("schedule", &Scheduler::Schedule, py::arg("now_ms") = 0)
      .def("micro_batch_of", &Scheduler::MicroBatchOf)
      .def("set_hold_waiting", &Scheduler::SetHoldWaiting)
      .def("set_paused", &Scheduler::SetPaused)
      .def(
          "pack",
          [](const Scheduler& s, const StepPlan& plan, py::array_t<int32_t, py::array::c_style> buf, int max_blocks) {
            auto info = buf.request(true);
            PackedLayout l = s.Pack(plan, static_cast<int32_t*>(info.ptr), info.size, max_blocks);
            if (l.total_words < 0) throw std::runtime_error("step staging buffer too small");
            py::dict d;
            d["num_seqs"] = l.num_seqs;
            d["num_prefill"] = l.num_prefill;
            d["num_decode"] = l.num_decode;
            d["total_tokens"] = l.total_tokens;
            d["total_logits"] = l.total_logits;
            d["max_q_len"] = l.max_q_len;
            d["max_kv_len"] = l.max_kv_len;
            d["max_blocks"] = l.max_blocks;
            d["input_ids"] = l.off_input_ids;
            d["positions"] = l.off_positions;
            d["slot_mapping"] = l.off_slot_mapping;
            d["seq_of_token"] = l.off_seq_of_token;
            d["cu_q"] = l.off_cu_q;
            d["kv_lens"] = l.off_kv_lens;
            d["q_starts"] = l.off_q_starts;
            d["logits_idx"] = l.off_logits_idx;
            d["block_tables"] = l.off_block_tables;
            d["total_words"] = l.total_words;
            return d;
          },
          py::arg("plan"), py::arg("buffer"), py::arg("max_blocks") = 0)
      .def("packed_words", &Scheduler::PackedWords)
      .def("update", &Scheduler::Update, py::arg("plan"), py::arg("sampled"), py::arg("now_ms") = 0)
      .def("resolve", &Scheduler::Resolve, py::arg("plan"), py::arg("real"))
      .def("set_micro_batch", &Scheduler::SetMicroBatch, py::arg("mb"), py::arg("count") = 1);

  py::class_<DraftTrie>(m, "DraftTrie")
      .def(py::init<int, int>(), py::arg("max_depth") = 16, py::arg("max_nodes") = 1 << 18)
      .def("feed", &DraftTrie::Feed)
      .def("feed_one", &DraftTrie::FeedOne)
      .def("propose", &DraftTrie::Propose, py::arg("num_draft"), py::arg("max_match") = 4, py::arg("min_match") = 1)
      .def_property_readonly("num_nodes", &DraftTrie::num_nodes);

  m.def("balance_workloads", &BalanceWorkloads);

  m.attr("RET_SUCCESS") = static_cast<int>(RET_SUCCESS);
  m.attr("RET_EXCEED_CAPACITY") = static_cast<int>(RET_EXCEED_CAPACITY);
  m.attr("RET_INPUT_LENGTH_EXCEEDED") = static_cast<int>(RET_INPUT_LENGTH_EXCEEDED);
  m.attr("RET_INVALID_ARGUMENT") = static_cast<int>(RET_INVALID_ARGUMENT);
  m.attr("RET_OUT_OF_MEMORY") = static_cast<int>(RET_OUT_OF_MEMORY);
  m.attr("FINISH_NONE") = static_cast<int>(FINISH_NONE);
  m.attr("FINISH_EOS") = static_cast<int>(FINISH_EOS);
  m.attr("FINISH_STOP_TOKEN") = static_cast<int>(FINISH_STOP_TOKEN);
  m.attr("FINISH_LENGTH") = static_cast<int>(FINISH_LENGTH);
  m.attr("FINISH_ABORTED") = static_cast<int>(FINISH_ABORTED);
  m.attr("FINISH_TIMEOUT") = static_cast<int>(FINISH_TIMEOUT);
  m.attr("FINISH_STOP_STRING") = static_cast<int>(FINISH_STOP_STRING);
  m.attr("FINISH_ERROR") = static_cast<int>(FINISH_ERROR);
}
