// Python bindings of the native host code: the cache manager and the scheduler.
// C++ exceptions map onto the classes of ferrum_b200.errors.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"
#include "step_plan.hpp"

namespace py = pybind11;
using namespace ferrum;

static void raise_as(const char* cls, const char* what) {
  py::object errors = py::module_::import("ferrum_b200.errors");
  PyErr_SetString(errors.attr(cls).ptr(), what);
}

PYBIND11_MODULE(_host, m) {
  m.doc() = "native cache manager and scheduler of ferrum_b200";
  m.attr("ABI") = 5;

  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const Unavailable& e) {
      raise_as("Unavailable", e.what());
    } catch (const CacheError& e) {
      raise_as("CacheError", e.what());
    } catch (const InvalidRequest& e) {
      raise_as("InvalidRequest", e.what());
    } catch (const NotFound& e) {
      raise_as("NotFound", e.what());
    } catch (const SchedulerError& e) {
      raise_as("SchedulerError", e.what());
    }
  });

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int page_size, int window, int num_pages, int table_width) {
             GroupSpec g;
             g.page_size = page_size;
             g.window = window;
             g.num_pages = num_pages;
             g.table_width = table_width;
             return g;
           }),
           py::arg("page_size"), py::arg("window"), py::arg("num_pages"), py::arg("table_width"))
      .def_readonly("page_size", &GroupSpec::page_size)
      .def_readonly("window", &GroupSpec::window)
      .def_readonly("num_pages", &GroupSpec::num_pages)
      .def_readonly("table_width", &GroupSpec::table_width);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupSpec>, int>(), py::arg("groups"), py::arg("max_requests"))
      .def_property_readonly("n_groups", &CacheManager::n_groups)
      .def_property_readonly("max_requests", &CacheManager::max_requests)
      .def("group", &CacheManager::group)
      .def("open", &CacheManager::open)
      .def("close", &CacheManager::close)
      .def("is_open", &CacheManager::is_open)
      .def("pages_missing", &CacheManager::pages_missing)
      .def("can_grow", &CacheManager::can_grow)
      .def("grow", &CacheManager::grow)
      .def("commit", &CacheManager::commit)
      .def("max_growable", &CacheManager::max_growable)
      .def("seq_len", &CacheManager::seq_len)
      .def("free_pages", &CacheManager::free_pages)
      .def("used_pages", &CacheManager::used_pages)
      .def("free_slots", &CacheManager::free_slots)
      .def("pages_held", &CacheManager::pages_held)
      .def("table", &CacheManager::table)
      .def("check", &CacheManager::check)
      .def("capacity_tokens", &CacheManager::capacity_tokens);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_batch_tokens", &SchedulerConfig::max_batch_tokens)
      .def_readwrite("max_batch_seqs", &SchedulerConfig::max_batch_seqs)
      .def_readwrite("chunk_size", &SchedulerConfig::chunk_size)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("n_vocab", &SchedulerConfig::n_vocab)
      .def_readwrite("eos_token_ids", &SchedulerConfig::eos_token_ids);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("id", &PlanEntry::id)
      .def_readonly("slot", &PlanEntry::slot)
      .def_readonly("pos0", &PlanEntry::pos0)
      .def_readonly("tokens", &PlanEntry::tokens)
      .def_readonly("sample", &PlanEntry::sample)
      .def_readonly("temperature", &PlanEntry::temperature)
      .def_readonly("seed", &PlanEntry::seed)
      .def_readonly("counter", &PlanEntry::counter)
      .def_readonly("from_device", &PlanEntry::from_device);

  py::class_<Event>(m, "Event")
      .def_readonly("kind", &Event::kind)
      .def_readonly("id", &Event::id)
      .def_readonly("token", &Event::token)
      .def_readonly("reason", &Event::reason);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("prompt_tokens", &SchedulerStats::prompt_tokens)
      .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("finished", &SchedulerStats::finished);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager*, SchedulerConfig>(), py::arg("cache"), py::arg("config"), py::keep_alive<1, 2>())
      .def("submit", &Scheduler::submit, py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("temperature") = 0.0f, py::arg("top_p") = 1.0f, py::arg("seed") = 0,
           py::arg("stop") = std::vector<int32_t>())
      .def("cancel", &Scheduler::cancel)
      .def("plan", &Scheduler::plan)
      .def("commit", &Scheduler::commit)
      .def("abandon", &Scheduler::abandon)
      .def("plan_ahead", &Scheduler::plan_ahead)
      .def("planned", &Scheduler::planned)
      .def("queued", &Scheduler::queued)
      .def("active", &Scheduler::active)
      .def("idle", &Scheduler::idle)
      .def("stats", &Scheduler::stats);

  py::class_<DecodePlan>(m, "DecodePlan")
      .def_readonly("n_items", &DecodePlan::n_items)
      .def_readonly("n_ctas", &DecodePlan::n_ctas)
      .def_readonly("n_slots", &DecodePlan::n_slots)
      .def_readonly("n_split_requests", &DecodePlan::n_split_requests);
  m.def("copy_tables", &copy_tables, py::arg("cache"), py::arg("group"), py::arg("slots"), py::arg("dst"),
        py::arg("row_stride"));
  m.def("build_decode_plan", &build_decode_plan, py::arg("kv_lo"), py::arg("kv_hi"), py::arg("n_kv_heads"),
        py::arg("cta_slots"), py::arg("min_tiles_per_cta"), py::arg("item_cap"), py::arg("cta_cap"), py::arg("pad"),
        py::arg("dst"));

  m.attr("FINISH_STOP") = (int)FINISH_STOP;
  m.attr("FINISH_LENGTH") = (int)FINISH_LENGTH;
  m.attr("FINISH_CANCELLED") = (int)FINISH_CANCELLED;
}
