// Python bindings of the host runtime (cache manager and scheduler).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace kvb;

PYBIND11_MODULE(_kvb_host, m) {
  m.doc() = "Host runtime: paged cache bookkeeping and the continuous-batching scheduler";

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int page_size, int window) { return GroupSpec{page_size, window}; }),
           py::arg("page_size"), py::arg("window") = 0)
      .def_readwrite("page_size", &GroupSpec::page_size)
      .def_readwrite("window", &GroupSpec::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupSpec>, std::vector<int>, int>(), py::arg("groups"),
           py::arg("pages_per_group"), py::arg("num_slots"))
      .def("admit", &CacheManager::admit)
      .def("has", &CacheManager::has)
      .def("slot_of", &CacheManager::slot_of)
      .def("computed", &CacheManager::computed)
      .def("pages_needed", &CacheManager::pages_needed)
      .def("extend", &CacheManager::extend)
      .def("advance", &CacheManager::advance)
      .def("release", &CacheManager::release)
      .def("drop_pages", &CacheManager::drop_pages)
      .def("block_table", &CacheManager::block_table)
      .def("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def("num_pages", &CacheManager::num_pages)
      .def("free_pages", &CacheManager::free_pages)
      .def("num_slots", &CacheManager::num_slots)
      .def("free_slots", &CacheManager::free_slots)
      .def("live_requests", &CacheManager::live_requests)
      .def("pages_taken_total", &CacheManager::pages_taken_total)
      .def("check", &CacheManager::check);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init([](int seqs, int tokens, int len, int chunk, int portions) {
             return SchedulerConfig{seqs, tokens, len, chunk, portions};
           }),
           py::arg("max_num_seqs"), py::arg("max_num_batched_tokens"), py::arg("max_model_len"),
           py::arg("max_prefill_chunk") = 0, py::arg("max_portions_per_step") = 0)
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("max_prefill_chunk", &SchedulerConfig::max_prefill_chunk)
      .def_readwrite("max_portions_per_step", &SchedulerConfig::max_portions_per_step);

  py::enum_<FinishReason>(m, "FinishReason")
      .value("NONE", FinishReason::None)
      .value("STOP", FinishReason::Stop)
      .value("LENGTH", FinishReason::Length)
      .value("MODEL_LEN", FinishReason::ModelLen)
      .value("CACHE_EXHAUSTED", FinishReason::CacheExhausted)
      .value("ABORTED", FinishReason::Aborted);
  m.def("finish_reason_name", &finish_reason_name);
  m.attr("PENDING_TOKEN") = kPendingToken;

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("id", &PlanEntry::id)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("tokens", &PlanEntry::tokens)
      .def_readonly("sample", &PlanEntry::sample);

  py::class_<Plan>(m, "Plan")
      .def_readonly("entries", &Plan::entries)
      .def_readonly("preempted", &Plan::preempted)
      .def_readonly("finished", &Plan::finished)
      .def_readonly("num_tokens", &Plan::num_tokens);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("scheduled_tokens", &SchedulerStats::scheduled_tokens)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("recomputed_tokens", &SchedulerStats::recomputed_tokens)
      .def_readonly("finished", &SchedulerStats::finished);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager*, SchedulerConfig>(), py::arg("cache"), py::arg("config"),
           py::keep_alive<1, 2>())
      .def("add", &Scheduler::add, py::arg("id"), py::arg("prompt"), py::arg("max_tokens"))
      .def("schedule", &Scheduler::schedule)
      .def("commit", &Scheduler::commit)
      .def("append_token", &Scheduler::append_token, py::arg("id"), py::arg("token"),
           py::arg("is_stop") = false)
      .def("mark_pending", &Scheduler::mark_pending)
      .def("resolve", &Scheduler::resolve, py::arg("id"), py::arg("token"), py::arg("is_stop") = false)
      .def("has_pending", &Scheduler::has_pending)
      .def("abort", &Scheduler::abort)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def("num_running", &Scheduler::num_running)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("is_live", &Scheduler::is_live)
      .def("is_finished", &Scheduler::is_finished)
      .def("tokens", &Scheduler::tokens)
      .def("prompt_len", &Scheduler::prompt_len)
      .def("output", &Scheduler::output)
      .def("finish_reason", &Scheduler::finish_reason)
      .def("preemptions_of", &Scheduler::preemptions_of)
      .def("take_finished", &Scheduler::take_finished)
      .def("stats", &Scheduler::stats)
      .def("config", &Scheduler::config);
}
