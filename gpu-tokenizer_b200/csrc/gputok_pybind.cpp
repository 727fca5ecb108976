// gputok_pybind.cpp -- Python module `gputok_gpu`: the reference's pybind
// surface (PYBIND11_MODULE(gputok_gpu, m), gputok_binding.cu:1015-1065) as a
// thin wrapper over the C ABI of include/gputok_b200.h.  No CUDA code here.
//
//   GpuTokenizer(merges_path, chunk_tokens=2048, max_iters=50, device=0)
//   .tokenize_batch(texts, merge_rule="greedy") -> (list[list[int]], kernel_ms)
//   .tokenize_batch_blockbpe_base(texts) -> (list[list[int]], kernel_ms)
//   .tokenize_batch_cpu(texts, merge_rule="greedy") -> list[list[int]]
// plus array-returning variants that skip the per-token Python objects:
//   .encode_packed(texts, mode="opt")    -> (ids int32[N], text_offsets int64[T+1],
//                                            chunk_offsets int64[C+1], kernel_ms)
//   .decode(ids) -> bytes, .table_info() -> dict, .stage_ms() -> dict
//
// Exceptions follow the reference: chunk_tokens <= 0 -> ValueError
// (std::invalid_argument, :661-663), unreadable/empty merges -> RuntimeError;
// CUDA failures raise RuntimeError instead of terminating the process (:24-30).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/gputok_b200.h"

namespace py = pybind11;

namespace {

[[noreturn]] void raise_status(int rc, const std::string& msg)
{
  if (rc == GTK_ERR_INVALID_ARG) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}

class GpuTokenizer {
 public:
  GpuTokenizer(const std::string& merges_path, int chunk_tokens, int max_iters, int device)
  {
    int rc = gtk_create(merges_path.c_str(), chunk_tokens, max_iters, device, &h_);
    if (rc != GTK_OK) raise_status(rc, gtk_global_error());
  }
  ~GpuTokenizer() { gtk_destroy(h_); }
  GpuTokenizer(const GpuTokenizer&) = delete;
  GpuTokenizer& operator=(const GpuTokenizer&) = delete;

  // Flatten list[str] into one byte buffer + offsets (UTF-8, as pybind's
  // str -> std::string caster does for the reference).
  static void flatten(const std::vector<std::string>& texts, std::vector<uint8_t>& bytes,
                      std::vector<int64_t>& off)
  {
    size_t total = 0;
    for (auto& t : texts) total += t.size();
    bytes.resize(total);
    off.assign(1, 0);
    off.reserve(texts.size() + 1);
    size_t k = 0;
    for (auto& t : texts) {
      if (!t.empty()) std::memcpy(bytes.data() + k, t.data(), t.size());
      k += t.size();
      off.push_back(int64_t(k));
    }
  }

  void check(int rc) const
  {
    if (rc != GTK_OK) raise_status(rc, gtk_last_error(h_));
  }

  // (list[list[int]], kernel_ms); ([], 0.0) for an empty batch or a batch of
  // empty texts, as gputok_binding.cpp:707-709, 734-736.
  py::tuple lists_from_result(size_t n_texts, float kernel_ms) const
  {
    int64_t n_ids = 0, n_chunks = 0;
    gtk_result_sizes(h_, &n_ids, &n_chunks, nullptr);
    py::list batch;
    if (n_texts == 0 || n_chunks == 0) return py::make_tuple(batch, 0.0);
    const int32_t* ids;
    const int64_t* toff;
    gtk_result_view(h_, &ids, &toff, nullptr);
    for (size_t t = 0; t < n_texts; ++t) {
      py::list one;
      for (int64_t i = toff[t]; i < toff[t + 1]; ++i) one.append(py::int_(ids[i]));
      batch.append(std::move(one));
    }
    return py::make_tuple(batch, double(kernel_ms));
  }

  py::tuple tokenize(const std::vector<std::string>& texts, int mode)
  {
    std::vector<uint8_t> bytes;
    std::vector<int64_t> off;
    flatten(texts, bytes, off);
    float ms = 0.f;
    int rc;
    {
      py::gil_scoped_release nogil;
      rc = gtk_encode(h_, mode, bytes.data(), off.data(), int64_t(texts.size()), &ms);
    }
    check(rc);
    return lists_from_result(texts.size(), ms);
  }

  py::list tokenize_cpu(const std::vector<std::string>& texts, const std::string& rule)
  {
    int r;
    if (rule == "greedy") r = GTK_RULE_GREEDY;
    else if (rule == "localmin") r = GTK_RULE_LOCALMIN;
    else throw std::invalid_argument("merge_rule must be 'greedy' or 'localmin'");
    std::vector<uint8_t> bytes;
    std::vector<int64_t> off;
    flatten(texts, bytes, off);
    int rc;
    {
      py::gil_scoped_release nogil;
      rc = gtk_encode_cpu(h_, r, bytes.data(), off.data(), int64_t(texts.size()));
    }
    check(rc);
    const int32_t* ids;
    const int64_t* toff;
    gtk_result_view(h_, &ids, &toff, nullptr);
    py::list batch;
    for (size_t t = 0; t < texts.size(); ++t) {
      py::list one;
      for (int64_t i = toff[t]; i < toff[t + 1]; ++i) one.append(py::int_(ids[i]));
      batch.append(std::move(one));
    }
    return batch;
  }

  py::tuple encode_packed(const std::vector<std::string>& texts, const std::string& mode)
  {
    int m;
    if (mode == "opt") m = GTK_MODE_OPT;
    else if (mode == "base") m = GTK_MODE_BASE;
    else throw std::invalid_argument("mode must be 'opt' or 'base'");
    std::vector<uint8_t> bytes;
    std::vector<int64_t> off;
    flatten(texts, bytes, off);
    float ms = 0.f;
    int rc;
    {
      py::gil_scoped_release nogil;
      rc = gtk_encode(h_, m, bytes.data(), off.data(), int64_t(texts.size()), &ms);
    }
    check(rc);
    int64_t n_ids = 0, n_chunks = 0;
    gtk_result_sizes(h_, &n_ids, &n_chunks, nullptr);
    py::array_t<int32_t> ids(n_ids);
    py::array_t<int64_t> toff(int64_t(texts.size()) + 1), coff(n_chunks + 1);
    check(gtk_result_copy(h_, ids.mutable_data(), n_ids, toff.mutable_data(), coff.mutable_data(), n_chunks + 1));
    return py::make_tuple(ids, toff, coff, double(ms));
  }

  py::bytes decode(const std::vector<int32_t>& ids) const
  {
    int64_t n = 0;
    check(gtk_decode(h_, ids.data(), int64_t(ids.size()), nullptr, 0, &n));
    std::string out(size_t(n), '\0');
    check(gtk_decode(h_, ids.data(), int64_t(ids.size()), reinterpret_cast<uint8_t*>(&out[0]), n, &n));
    return py::bytes(out);
  }

  py::dict table_info() const
  {
    gtk_table_info ti;
    check(gtk_table_info_get(h_, &ti));
    py::dict d;
    d["vocab_size"] = ti.vocab_size;
    d["num_merges"] = ti.num_merges;
    d["max_rank"] = ti.max_rank;
    d["hash_capacity"] = ti.hash_capacity;
    d["hash_overflow_entries"] = ti.hash_overflow_entries;
    d["hash_bytes"] = ti.hash_bytes;
    d["monotone"] = bool(ti.monotone);
    d["merged_is_256_plus_rank"] = bool(ti.merged_is_256_plus_rank);
    d["byte_ids_identity"] = bool(ti.byte_ids_identity);
    d["adj_bigrams"] = ti.adj_bigrams;
    d["chunk_tokens"] = ti.chunk_tokens;
    d["max_iters"] = ti.max_iters;
    d["device"] = ti.device;
    d["sm_count"] = ti.sm_count;
    d["whole_segment_entries"] = ti.whole_segment_entries;
    d["whole_segment_dropped"] = ti.whole_segment_dropped;
    return d;
  }

  void set_stage_timing(bool per_stage) { check(gtk_set_stage_timing(h_, per_stage ? 1 : 0)); }

  py::dict stage_ms() const
  {
    float ms[5];
    int32_t launches = 0;
    check(gtk_last_stage_ms(h_, ms, &launches));
    py::dict d;
    d["chunker"] = ms[0];
    d["merge"] = ms[1];
    d["scan"] = ms[2];
    d["pack"] = ms[3];
    d["pipeline"] = ms[4];
    d["kernel_launches"] = launches;
    return d;
  }

 private:
  gtk_tokenizer* h_ = nullptr;
};

}  // namespace

PYBIND11_MODULE(gputok_gpu, m)
{
  m.doc() = "B200-native greedy byte-level BPE tokenizer (drop-in for the reference's gputok_gpu module)";
  m.attr("__version__") = gtk_version();

  py::class_<GpuTokenizer>(m, "GpuTokenizer")
    .def(py::init<const std::string&, int, int, int>(), py::arg("merges_path"), py::arg("chunk_tokens") = 2048,
         py::arg("max_iters") = 50, py::arg("device") = 0)
    .def("tokenize_batch", [](GpuTokenizer& self, const std::vector<std::string>& texts, const std::string& rule) {
           if (rule == "greedy") return self.tokenize(texts, GTK_MODE_OPT);
           if (rule == "localmin") return self.tokenize(texts, GTK_MODE_LOCALMIN);
           throw std::invalid_argument("merge_rule must be 'greedy' or 'localmin'");
         }, py::arg("texts"), py::arg("merge_rule") = "greedy",
         "Tokenize a batch of UTF-8 strings with the segment-parallel kernel (greedy rule).\n"
         "merge_rule='localmin' runs the reference method's own rule (local minimum, max_iters passes,\n"
         "per chunk) on the GPU instead.  Returns (list[list[int]], kernel_time_ms).")
    .def("tokenize_batch_blockbpe_base", [](GpuTokenizer& self, const std::vector<std::string>& texts) {
           return self.tokenize(texts, GTK_MODE_BASE);
         }, py::arg("texts"),
         "Tokenize with the one-CTA-per-chunk Algorithm 1 kernel.\n"
         "Returns (list[list[int]], kernel_time_ms).")
    .def("tokenize_batch_cpu", &GpuTokenizer::tokenize_cpu, py::arg("texts"), py::arg("merge_rule") = "greedy",
         "Host reference tokenizer. merge_rule='greedy' (default) is the rule the GPU paths\n"
         "implement, per chunk; 'localmin' is the reference method's own rule on the whole text.")
    .def("encode_packed", &GpuTokenizer::encode_packed, py::arg("texts"), py::arg("mode") = "opt",
         "Returns (ids int32[N], text_offsets int64[T+1], chunk_offsets int64[C+1], kernel_time_ms).")
    .def("decode", &GpuTokenizer::decode, py::arg("ids"))
    .def("table_info", &GpuTokenizer::table_info)
    .def("stage_ms", &GpuTokenizer::stage_ms)
    .def("set_stage_timing", [](GpuTokenizer& self, bool per_stage) { self.set_stage_timing(per_stage); },
         py::arg("per_stage"),
         "Time every stage of a batch (stage_ms()['chunker'/'merge'/'scan'/'pack']) instead of the pipeline as a\n"
         "whole; off by default.");
}
