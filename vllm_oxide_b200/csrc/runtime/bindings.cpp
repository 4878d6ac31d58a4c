// Python bindings of the host runtime: cache manager, step-batch builder, scheduler.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/numpy.h>
#include "scheduler.h"

namespace py = pybind11;
using namespace vob;

static py::dict layout_dict(const StepLayout& L) {
    py::dict d;
    d["rows_cap"] = L.rows_cap; d["seqs_cap"] = L.seqs_cap; d["logits_cap"] = L.logits_cap;
    d["groups"] = L.groups; d["max_pages"] = L.max_pages;
    d["tokens"] = L.tokens; d["positions"] = L.positions; d["row_seq"] = L.row_seq;
    d["seq_starts"] = L.seq_starts; d["context_lens"] = L.context_lens; d["seq_lens"] = L.seq_lens;
    d["state_slots"] = L.state_slots; d["logit_rows"] = L.logit_rows; d["temperature"] = L.temperature;
    d["seeds"] = L.seeds; d["sample_steps"] = L.sample_steps;
    d["slot_mapping"] = L.slot_mapping; d["block_tables"] = L.block_tables; d["total"] = L.total;
    return d;
}

PYBIND11_MODULE(VOB_MODULE_NAME, m) {
    m.doc() = "host runtime: paged-cache bookkeeping, step batches, scheduler";
    py::register_exception<CacheError>(m, "RuntimeFault");

    py::class_<GroupSpec>(m, "GroupSpec")
        .def(py::init([](int kind, int window, int num_pages) { GroupSpec g; g.kind = kind; g.window = window; g.num_pages = num_pages; return g; }),
             py::arg("kind"), py::arg("window"), py::arg("num_pages"))
        .def_readwrite("kind", &GroupSpec::kind)
        .def_readwrite("window", &GroupSpec::window)
        .def_readwrite("num_pages", &GroupSpec::num_pages);
    m.attr("FULL") = (int)kFull;
    m.attr("WINDOW") = (int)kWindow;

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<int, std::vector<GroupSpec>, int>(), py::arg("page_size"), py::arg("groups"), py::arg("num_state_slots"))
        .def_property_readonly("page_size", &CacheManager::page_size)
        .def_property_readonly("num_groups", &CacheManager::num_groups)
        .def_property_readonly("num_state_slots", &CacheManager::num_state_slots)
        .def("group", &CacheManager::group)
        .def("num_free_pages", &CacheManager::num_free_pages)
        .def("num_pages", &CacheManager::num_pages)
        .def("num_free_slots", &CacheManager::num_free_slots)
        .def("num_requests", &CacheManager::num_requests)
        .def("has", &CacheManager::has)
        .def("admit", &CacheManager::admit)
        .def("reserve", &CacheManager::reserve)
        .def("tokens_that_fit", &CacheManager::tokens_that_fit)
        .def("max_pages_held", &CacheManager::max_pages_held)
        .def("first_visible", &CacheManager::first_visible)
        .def("commit", &CacheManager::commit)
        .def("release", &CacheManager::release)
        .def("slot_of", &CacheManager::slot_of)
        .def("length", [](const CacheManager& c, int64_t id) { return c.get(id).len; })
        .def("state_slot", [](const CacheManager& c, int64_t id) { return c.get(id).slot; })
        .def("block_table", [](const CacheManager& c, int64_t id, int g) { return c.get(id).tables.at(g); })
        .def("check_invariants", &CacheManager::check_invariants);

    py::class_<StepEntry>(m, "StepEntry")
        .def(py::init([](int64_t id, std::vector<int32_t> tokens, std::vector<int32_t> want, float temperature,
                         uint64_t seed, int sample_step) {
                 StepEntry e; e.id = id; e.tokens = std::move(tokens); e.want = std::move(want);
                 e.temperature = temperature; e.seed = seed; e.sample_step = sample_step; return e; }),
             py::arg("id"), py::arg("tokens"), py::arg("want") = std::vector<int32_t>{}, py::arg("temperature") = 0.f,
             py::arg("seed") = 0, py::arg("sample_step") = 0)
        .def_readwrite("id", &StepEntry::id)
        .def_readwrite("tokens", &StepEntry::tokens)
        .def_readwrite("want", &StepEntry::want);

    py::class_<StepArrays>(m, "StepArrays")
        .def_readonly("rows", &StepArrays::rows)
        .def_readonly("seqs", &StepArrays::seqs)
        .def_readonly("logit_count", &StepArrays::logit_count)
        .def_readonly("max_new", &StepArrays::max_new)
        .def_readonly("lead_single", &StepArrays::lead_single)
        .def_readonly("max_seq_len", &StepArrays::max_seq_len)
        .def_readonly("any_sampling", &StepArrays::any_sampling)
        .def_readonly("ids", &StepArrays::ids)
        .def_readonly("new_counts", &StepArrays::new_counts)
        .def_property_readonly("layout", [](const StepArrays& a) { return layout_dict(a.layout); })
        .def_property_readonly("total", [](const StepArrays& a) { return a.layout.total; })
        .def_readonly("used", &StepArrays::used)
        // Copy the packed int32 buffer into a caller-owned (pinned) array of at least `total` ints.
        .def("copy_into", [](const StepArrays& a, py::array_t<int32_t, py::array::c_style> dst) {
            if ((size_t)dst.size() < (size_t)a.used) throw CacheError("copy_into: destination too small");
            std::memcpy(dst.mutable_data(), a.data.data(), (size_t)a.used * sizeof(int32_t));
        })
        .def("data", [](const StepArrays& a) {
            return py::array_t<int32_t>((py::ssize_t)a.data.size(), a.data.data());
        });

    m.def("step_layout", [](int rows_cap, int seqs_cap, int logits_cap, int groups, int max_pages) {
        return layout_dict(StepLayout::make(rows_cap, seqs_cap, logits_cap, groups, max_pages));
    });
    m.def("build_step", &build_step, py::arg("cache"), py::arg("entries"), py::arg("rows_cap"), py::arg("seqs_cap"),
          py::arg("logits_cap"), py::arg("max_pages"), py::arg("vocab_size"));

    py::class_<SamplingParams>(m, "SamplingParams")
        .def(py::init([](int max_new_tokens, float temperature, uint64_t seed, std::vector<int32_t> stop) {
                 SamplingParams p; p.max_new_tokens = max_new_tokens; p.temperature = temperature; p.seed = seed;
                 p.stop_token_ids = std::move(stop); return p; }),
             py::arg("max_new_tokens") = 16, py::arg("temperature") = 0.f, py::arg("seed") = 0,
             py::arg("stop_token_ids") = std::vector<int32_t>{})
        .def_readwrite("max_new_tokens", &SamplingParams::max_new_tokens)
        .def_readwrite("temperature", &SamplingParams::temperature)
        .def_readwrite("seed", &SamplingParams::seed)
        .def_readwrite("stop_token_ids", &SamplingParams::stop_token_ids);

    py::class_<PlannedEntry>(m, "PlannedEntry")
        .def_readonly("id", &PlannedEntry::id)
        .def_readonly("start", &PlannedEntry::start)
        .def_readonly("count", &PlannedEntry::count)
        .def_readonly("sample", &PlannedEntry::sample);

    py::class_<StepPlan>(m, "StepPlan")
        .def_readonly("entries", &StepPlan::entries)
        .def_property_readonly("num_entries", [](const StepPlan& p) { return p.entries.size(); })
        .def_property_readonly("decode_only", &StepPlan::decode_only)
        .def("sampling_ids", &StepPlan::sampling_ids)
        .def_readonly("preempted", &StepPlan::preempted)
        .def_readonly("admitted", &StepPlan::admitted)
        .def_readonly("failed", &StepPlan::failed);

    py::class_<Finished>(m, "Finished")
        .def_readonly("id", &Finished::id)
        .def_readonly("reason", &Finished::reason)
        .def_readonly("output", &Finished::output);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<CacheManager*, int, int, int, int>(), py::arg("cache"), py::arg("max_batch_tokens"),
             py::arg("max_seqs"), py::arg("max_model_len"), py::arg("prefill_chunk") = 0, py::keep_alive<1, 2>())
        .def("add_request", &Scheduler::add_request)
        .def("set_admission_watermark", &Scheduler::set_admission_watermark)
        .def("admission_watermark", &Scheduler::admission_watermark)
        .def("has_unfinished", &Scheduler::has_unfinished)
        .def("num_waiting", &Scheduler::num_waiting)
        .def("num_running", &Scheduler::num_running)
        .def("running", &Scheduler::running)
        .def("waiting", &Scheduler::waiting)
        .def("schedule", &Scheduler::schedule)
        .def("arrays", &Scheduler::arrays)
        .def("update", &Scheduler::update)
        .def("steady_decode", &Scheduler::steady_decode)
        .def("advance", &Scheduler::advance)
        .def("resolve", &Scheduler::resolve)
        .def("take_done", &Scheduler::take_done)
        .def("abort", &Scheduler::abort)
        .def("tokens_of", [](const Scheduler& s, int64_t id) { return s.request(id).tokens; })
        .def("computed_of", [](const Scheduler& s, int64_t id) { return s.request(id).computed; })
        .def("preemptions_of", [](const Scheduler& s, int64_t id) { return s.request(id).preemptions; });
}
