// pybind11 surface of the host runtime: CacheManager and Scheduler.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace vcb;

PYBIND11_MODULE(_vcb_runtime, m) {
    m.doc() = "Host runtime: page pools, block tables, state slots, continuous-batching scheduler";
    py::register_exception<CacheError>(m, "CacheError", PyExc_RuntimeError);

    py::class_<GroupSpec>(m, "GroupSpec")
        .def(py::init([](int32_t page_size, int32_t num_pages, int32_t window) {
                 GroupSpec g;
                 g.page_size = page_size;
                 g.num_pages = num_pages;
                 g.window = window;
                 return g;
             }),
             py::arg("page_size"), py::arg("num_pages"), py::arg("window") = 0)
        .def_readwrite("page_size", &GroupSpec::page_size)
        .def_readwrite("num_pages", &GroupSpec::num_pages)
        .def_readwrite("window", &GroupSpec::window);

    py::class_<IdPool>(m, "IdPool")
        .def(py::init<int32_t>())
        .def("alloc",
             [](IdPool& p, int32_t n) -> py::object {
                 std::vector<int32_t> out;
                 if (!p.alloc(n, out)) return py::none();
                 return py::cast(out);
             })
        .def("free", &IdPool::free)
        .def("free_count", &IdPool::free_count)
        .def("size", &IdPool::size)
        .def("is_held", &IdPool::is_held);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<std::vector<GroupSpec>, int32_t>(), py::arg("groups"), py::arg("num_slots"))
        .def("open", &CacheManager::open)
        .def("reserve", &CacheManager::reserve)
        .def("commit", &CacheManager::commit)
        .def("close", &CacheManager::close)
        .def("is_open", &CacheManager::is_open)
        .def("slot", &CacheManager::slot)
        .def("num_tokens", &CacheManager::num_tokens)
        .def("reserved_tokens", &CacheManager::reserved_tokens)
        .def("block_table", &CacheManager::block_table)
        .def("num_groups", &CacheManager::num_groups)
        .def("group", &CacheManager::group)
        .def("free_pages", &CacheManager::free_pages)
        .def("free_slots", &CacheManager::free_slots)
        .def("num_open", &CacheManager::num_open)
        .def("pages_missing", &CacheManager::pages_missing)
        .def("peak_pages", &CacheManager::peak_pages)
        .def("check_invariants", &CacheManager::check_invariants);

    py::enum_<RequestState>(m, "RequestState")
        .value("WAITING", RequestState::WAITING)
        .value("RUNNING", RequestState::RUNNING)
        .value("FINISHED", RequestState::FINISHED)
        .value("PREEMPTED", RequestState::PREEMPTED);

    py::class_<SamplingParams>(m, "SamplingParams")
        .def(py::init([](float temperature, float top_p, float repeat_penalty, uint64_t seed) {
                 SamplingParams s;
                 s.temperature = temperature;
                 s.top_p = top_p;
                 s.repeat_penalty = repeat_penalty;
                 s.seed = seed;
                 return s;
             }),
             py::arg("temperature") = 0.7f, py::arg("top_p") = 0.8f, py::arg("repeat_penalty") = 1.1f,
             py::arg("seed") = 0)
        .def_readwrite("temperature", &SamplingParams::temperature)
        .def_readwrite("top_p", &SamplingParams::top_p)
        .def_readwrite("repeat_penalty", &SamplingParams::repeat_penalty)
        .def_readwrite("seed", &SamplingParams::seed);

    py::class_<Request>(m, "Request")
        .def_readonly("id", &Request::id)
        .def_readonly("prompt", &Request::prompt)
        .def_readonly("generated", &Request::generated)
        .def_readonly("state", &Request::state)
        .def_readonly("max_new_tokens", &Request::max_new_tokens)
        .def_readonly("sampling", &Request::sampling)
        .def_readonly("stop_ids", &Request::stop_ids)
        .def_readonly("num_computed", &Request::num_computed)
        .def_readonly("slot", &Request::slot)
        .def_readonly("preempt_count", &Request::preempt_count)
        .def_readonly("finish_reason", &Request::finish_reason)
        .def("seq_len", &Request::seq_len);

    py::class_<ScheduledEntry>(m, "ScheduledEntry")
        .def_readonly("request", &ScheduledEntry::request)
        .def_readonly("slot", &ScheduledEntry::slot)
        .def_readonly("start_pos", &ScheduledEntry::start_pos)
        .def_readonly("tokens", &ScheduledEntry::tokens)
        .def_readonly("sample", &ScheduledEntry::sample)
        .def_readonly("gen_step", &ScheduledEntry::gen_step)
        .def_readonly("is_prompt", &ScheduledEntry::is_prompt);

    py::class_<SchedulerOutput>(m, "SchedulerOutput")
        .def_readonly("entries", &SchedulerOutput::entries)
        .def_readonly("preempted", &SchedulerOutput::preempted)
        .def_readonly("num_prompt_tokens", &SchedulerOutput::num_prompt_tokens)
        .def_readonly("num_generation_tokens", &SchedulerOutput::num_generation_tokens);

    py::class_<SchedulerStats>(m, "SchedulerStats")
        .def_readonly("steps", &SchedulerStats::steps)
        .def_readonly("preemptions", &SchedulerStats::preemptions)
        .def_readonly("recomputed_tokens", &SchedulerStats::recomputed_tokens)
        .def_readonly("prompt_tokens", &SchedulerStats::prompt_tokens)
        .def_readonly("generated_tokens", &SchedulerStats::generated_tokens);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<std::vector<GroupSpec>, int32_t, int32_t, int32_t>(), py::arg("groups"),
             py::arg("max_num_seqs"), py::arg("max_step_tokens"), py::arg("max_model_len"))
        .def("submit", &Scheduler::submit, py::arg("prompt"), py::arg("max_new_tokens"), py::arg("sampling"),
             py::arg("stop_ids") = std::vector<int32_t>{})
        .def("schedule", &Scheduler::schedule)
        .def("update", &Scheduler::update)
        .def("abort", &Scheduler::abort)
        .def("forget", &Scheduler::forget)
        .def("has_unfinished", &Scheduler::has_unfinished)
        .def("request", &Scheduler::request, py::return_value_policy::copy)
        .def("knows", &Scheduler::knows)
        .def("num_waiting", &Scheduler::num_waiting)
        .def("num_running", &Scheduler::num_running)
        .def("num_finished", &Scheduler::num_finished)
        .def("stats", &Scheduler::stats, py::return_value_policy::copy)
        .def("cache", py::overload_cast<>(&Scheduler::cache), py::return_value_policy::reference_internal)
        .def_property_readonly("max_step_tokens", &Scheduler::max_step_tokens)
        .def_property_readonly("max_num_seqs", &Scheduler::max_num_seqs)
        .def_property_readonly("max_model_len", &Scheduler::max_model_len);
}
