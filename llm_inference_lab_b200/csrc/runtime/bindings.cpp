// Python bindings of the host runtime (cache manager and scheduler).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace lab;

PYBIND11_MODULE(_lab_runtime, m) {
  m.doc() = "Host runtime: paged cache manager and scheduler";

  py::register_exception<CapacityError>(m, "CapacityError", PyExc_RuntimeError);
  py::register_exception<StateError>(m, "StateError", PyExc_RuntimeError);

  py::class_<GroupConfig>(m, "GroupConfig")
      .def(py::init([](int page_size, int window, int num_pages) {
             GroupConfig g;
             g.page_size = page_size;
             g.window = window;
             g.num_pages = num_pages;
             return g;
           }),
           py::arg("page_size"), py::arg("window"), py::arg("num_pages"))
      .def_readonly("page_size", &GroupConfig::page_size)
      .def_readonly("window", &GroupConfig::window)
      .def_readonly("num_pages", &GroupConfig::num_pages);

  py::class_<StepLayout>(m, "StepLayout")
      .def_readonly("tokens_cap", &StepLayout::tokens_cap)
      .def_readonly("requests_cap", &StepLayout::requests_cap)
      .def_readonly("table_width", &StepLayout::table_width)
      .def_readonly("row_req", &StepLayout::row_req)
      .def_readonly("row_pos", &StepLayout::row_pos)
      .def_readonly("q_start", &StepLayout::q_start)
      .def_readonly("kv_len", &StepLayout::kv_len)
      .def_readonly("pos0", &StepLayout::pos0)
      .def_readonly("state_slot", &StepLayout::state_slot)
      .def_readonly("row_slot", &StepLayout::row_slot)
      .def_readonly("block_table", &StepLayout::block_table)
      .def_readonly("total", &StepLayout::total);

  py::class_<CacheManager, std::shared_ptr<CacheManager>>(m, "CacheManager")
      .def(py::init<std::vector<GroupConfig>, int>(), py::arg("groups"), py::arg("max_requests"))
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def_property_readonly("max_requests", &CacheManager::max_requests)
      .def("has", &CacheManager::has)
      .def("free_pages", &CacheManager::free_pages)
      .def("used_pages", &CacheManager::used_pages)
      .def_property_readonly("free_state_slots", &CacheManager::free_state_slots)
      .def_property_readonly("used_state_slots", &CacheManager::used_state_slots)
      .def_property_readonly("live_requests", &CacheManager::live_requests)
      .def("open", &CacheManager::open)
      .def("length", [](const CacheManager& c, int64_t id) { return c.get(id).committed; })
      .def("reserved", [](const CacheManager& c, int64_t id) { return c.get(id).reserved; })
      .def("state_slot", [](const CacheManager& c, int64_t id) { return c.get(id).state_slot; })
      .def("pages_needed", &CacheManager::pages_needed)
      .def("pages_at_peak", &CacheManager::pages_at_peak)
      .def("can_reserve",
           [](const CacheManager& c, const std::vector<std::pair<int64_t, int>>& entries) {
             std::vector<StepEntry> e;
             for (auto& p : entries) e.push_back({p.first, p.second});
             return c.can_reserve(e);
           })
      .def("reserve", &CacheManager::reserve)
      .def("commit", &CacheManager::commit)
      .def("rollback", &CacheManager::rollback)
      .def("close", &CacheManager::close)
      .def("block_table", &CacheManager::block_table)
      .def("held_pages", &CacheManager::held_pages)
      .def("check_consistency", &CacheManager::check_consistency)
      .def("layout", &CacheManager::layout, py::arg("tokens_cap"), py::arg("requests_cap"), py::arg("table_width"))
      .def(
          "pack",
          [](const CacheManager& c, const std::vector<std::pair<int64_t, int>>& entries, const StepLayout& L,
             py::array_t<int32_t, py::array::c_style> buf, int pad_tokens, int pad_requests) {
            if (buf.size() < L.total) throw std::invalid_argument("staging buffer smaller than the layout");
            std::vector<StepEntry> e;
            for (auto& p : entries) e.push_back({p.first, p.second});
            c.pack(e, L, buf.mutable_data(), pad_tokens, pad_requests);
          },
          py::arg("entries"), py::arg("layout"), py::arg("buffer"), py::arg("pad_tokens") = 0,
          py::arg("pad_requests") = 0);

  py::enum_<FinishReason>(m, "FinishReason")
      .value("none", FinishReason::kNone)
      .value("length", FinishReason::kLength)
      .value("eos", FinishReason::kEos)
      .value("capacity", FinishReason::kCapacity)
      .value("invalid", FinishReason::kInvalid)
      .value("cancelled", FinishReason::kCancelled);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("id", &PlanEntry::id)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("n", &PlanEntry::n)
      .def_readonly("sample", &PlanEntry::sample)
      .def("__repr__", [](const PlanEntry& e) {
        return "PlanEntry(id=" + std::to_string(e.id) + ", start=" + std::to_string(e.start) +
               ", n=" + std::to_string(e.n) + ", sample=" + (e.sample ? "True" : "False") + ")";
      });

  py::class_<Finished>(m, "Finished")
      .def_readonly("id", &Finished::id)
      .def_readonly("generated", &Finished::generated)
      .def_readonly("reason", &Finished::reason)
      .def_readonly("prompt_len", &Finished::prompt_len)
      .def_readonly("preemptions", &Finished::preemptions)
      .def_readonly("message", &Finished::message);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init([](std::shared_ptr<CacheManager> cache, int max_batch_tokens, int max_seq_len, int max_active,
                       bool reserve_future) {
             SchedulerConfig cfg;
             cfg.max_batch_tokens = max_batch_tokens;
             cfg.max_seq_len = max_seq_len;
             cfg.max_active = max_active;
             cfg.reserve_future = reserve_future;
             return new Scheduler(std::move(cache), cfg);
           }),
           py::arg("cache"), py::arg("max_batch_tokens") = 512, py::arg("max_seq_len") = 0, py::arg("max_active") = 0,
           py::arg("reserve_future") = true)
      .def("add", &Scheduler::add, py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens") = 1,
           py::arg("eos") = std::vector<int>{}, py::arg("ignore_eos") = false)
      .def("cancel", &Scheduler::cancel)
      .def_property_readonly("idle", &Scheduler::idle)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_active", &Scheduler::num_active)
      .def_property_readonly("preemptions", &Scheduler::preemptions)
      .def("plan", &Scheduler::plan)
      .def("plan_ahead", &Scheduler::plan_ahead)
      .def("portion", &Scheduler::portion)
      .def("complete", &Scheduler::complete)
      .def("abandon", &Scheduler::abandon)
      .def("take_finished", &Scheduler::take_finished)
      .def("tokens", [](const Scheduler& s, int64_t id) { return s.find_active(id).tokens; })
      .def("is_decoding", [](const Scheduler& s, int64_t id) { return s.find_active(id).decoding; });
}
