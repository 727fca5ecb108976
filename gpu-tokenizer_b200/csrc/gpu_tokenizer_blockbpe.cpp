// gpu_tokenizer_blockbpe -- command-line front end with the arguments, output lines and output file
// of the reference's standalone binary (main() of gputok_blockbpe.cu:577-880), on top of the C ABI.
//
//   gpu_tokenizer_blockbpe [chunk_tokens=2048] [input_path=data/input/pride_and_prejudice.txt] [base|opt]
//
// Reads data/gpt2_tokenizer/merges.txt (as the reference does; GTK_MERGES overrides), tokenises the
// whole file as one text cut into chunks, runs the host greedy reference and the GPU path, compares
// them per chunk, prints the timing lines the reference's scripts parse
// (benchmark_tokenizer_scaling.py:155-157, profile_blockbpe_block_sizes.sh:30-32) and writes
// data/output/gpu_tokens_blockbpe.txt (GTK_OUTPUT overrides).  Exit code 0 iff CPU and GPU agree.
// The third argument picks the kernel: "base" (default, one CTA per chunk) or "opt".  GTK_BLOCK_SIZE=128|256|512|1024
// sets the threads per CTA of the base kernel, which the reference fixes at compile time (-DBLOCK_SIZE, :313-315).
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/gputok_b200.h"

int main(int argc, char** argv)
{
  const char* env_merges = std::getenv("GTK_MERGES");
  const char* env_output = std::getenv("GTK_OUTPUT");
  const std::string merges_path = env_merges ? env_merges : "data/gpt2_tokenizer/merges.txt";
  const std::string out_path    = env_output ? env_output : "data/output/gpu_tokens_blockbpe.txt";
  std::string input_path        = "data/input/pride_and_prejudice.txt";

  int chunk_tokens = 2048;
  if (argc > 1) {
    char* end = nullptr;
    long v    = std::strtol(argv[1], &end, 10);
    if (end == argv[1]) std::cerr << "Warning: failed to parse chunk size from argv[1]; using default " << chunk_tokens << std::endl;
    else chunk_tokens = int(std::max<long>(1, v));
  }
  if (argc > 2) input_path = argv[2];
  const int mode = (argc > 3 && std::strcmp(argv[3], "opt") == 0) ? GTK_MODE_OPT : GTK_MODE_BASE;

  gtk_tokenizer* tok = nullptr;
  int rc = gtk_create(merges_path.c_str(), chunk_tokens, 50, 0, &tok);
  if (rc != GTK_OK) {
    std::cerr << "Exception: " << gtk_global_error() << std::endl;
    return 1;
  }
  if (const char* bs = std::getenv("GTK_BLOCK_SIZE")) {
    if (gtk_set_base_block_size(tok, std::atoi(bs)) != GTK_OK) {
      std::cerr << "Exception: " << gtk_last_error(tok) << std::endl;
      return 1;
    }
  }
  gtk_table_info info;
  gtk_table_info_get(tok, &info);
  std::cerr << "Loaded BPE merges: " << info.num_merges << ", vocab size: " << info.vocab_size << std::endl;

  std::ifstream in(input_path, std::ios::binary);
  if (!in) {
    std::cerr << "Failed to open input file: " << input_path << std::endl;
    return 1;
  }
  std::ostringstream oss;
  oss << in.rdbuf();
  const std::string text = oss.str();
  if (text.empty()) {
    std::cerr << "Input file is empty: " << input_path << std::endl;
    return 0;
  }
  const int64_t total_tokens = int64_t(text.size());  // one initial token per byte
  const int64_t offsets[2]   = {0, total_tokens};
  const int64_t n_chunks_in  = (total_tokens + chunk_tokens - 1) / chunk_tokens;
  std::cerr << "Tokenized full text into " << n_chunks_in << " chunk(s), max tokens per chunk: "
            << std::min<int64_t>(chunk_tokens, total_tokens) << std::endl;
  std::cerr << "Total initial tokens: " << total_tokens << std::endl;

  // host greedy reference, timed as the reference times its CPU loop (:722-729)
  const auto t0 = std::chrono::high_resolution_clock::now();
  rc = gtk_encode_cpu(tok, GTK_RULE_GREEDY, reinterpret_cast<const uint8_t*>(text.data()), offsets, 1);
  const auto t1 = std::chrono::high_resolution_clock::now();
  if (rc != GTK_OK) {
    std::cerr << "Exception: " << gtk_last_error(tok) << std::endl;
    return 1;
  }
  const double cpu_ms = std::chrono::duration_cast<std::chrono::microseconds>(t1 - t0).count() / 1000.0;
  int64_t n_cpu = 0, c_cpu = 0;
  gtk_result_sizes(tok, &n_cpu, &c_cpu, nullptr);
  std::vector<int32_t> cpu_ids(size_t(n_cpu) + 1);
  std::vector<int64_t> cpu_off(size_t(c_cpu) + 1);
  gtk_result_copy(tok, cpu_ids.data(), n_cpu, nullptr, cpu_off.data(), c_cpu + 1);

  float gpu_ms = 0.f;
  rc = gtk_encode(tok, mode, reinterpret_cast<const uint8_t*>(text.data()), offsets, 1, &gpu_ms);  // warm-up
  if (rc == GTK_OK) rc = gtk_encode(tok, mode, reinterpret_cast<const uint8_t*>(text.data()), offsets, 1, &gpu_ms);
  if (rc != GTK_OK) {
    std::cerr << "CUDA error (" << gtk_last_error(tok) << ")" << std::endl;
    return 1;
  }
  int64_t n_gpu = 0, c_gpu = 0;
  gtk_result_sizes(tok, &n_gpu, &c_gpu, nullptr);
  const int32_t* gpu_ids;
  const int64_t* gpu_off;
  gtk_result_view(tok, &gpu_ids, nullptr, &gpu_off);

  bool all_ok = (c_cpu == c_gpu);
  if (!all_ok) std::cerr << "Chunk count mismatch: CPU " << c_cpu << " vs GPU " << c_gpu << std::endl;
  for (int64_t c = 0; all_ok && c < c_cpu; ++c) {
    const int64_t lc = cpu_off[c + 1] - cpu_off[c], lg = gpu_off[c + 1] - gpu_off[c];
    if (lc != lg) {
      all_ok = false;
      std::cerr << "[Seq " << c << "] Length mismatch: CPU " << lc << " vs GPU " << lg << std::endl;
      break;
    }
    for (int64_t j = 0; j < lc; ++j) {
      if (cpu_ids[cpu_off[c] + j] != gpu_ids[gpu_off[c] + j]) {
        all_ok = false;
        std::cerr << "[Seq " << c << "] Token mismatch at position " << j << ": CPU " << cpu_ids[cpu_off[c] + j]
                  << " vs GPU " << gpu_ids[gpu_off[c] + j] << std::endl;
        break;
      }
    }
  }

  std::cout << "CPU BPE (greedy Algorithm 1) time: " << cpu_ms << " ms" << std::endl;
  std::cout << "GPU BlockBPE-style greedy kernel time (excl. H2D/D2H): " << gpu_ms << " ms" << std::endl;
  if (gpu_ms > 0.0f) {
    std::cout << "Approximate speedup (CPU / GPU greedy kernel): " << cpu_ms / gpu_ms << "x" << std::endl;
    std::cout << "CPU throughput: " << double(total_tokens) / (cpu_ms / 1000.0) << " tokens/s" << std::endl;
    std::cout << "GPU greedy kernel throughput: " << double(total_tokens) / (gpu_ms / 1000.0) << " tokens/s" << std::endl;
  }
  std::cout << "CPU vs GPU token match (greedy Algorithm 1): " << (all_ok ? "OK" : "MISMATCH") << std::endl;

  if (gtk_write_token_strings(tok, out_path.c_str(), gpu_ids, gpu_off, c_gpu) != GTK_OK)
    std::cerr << "Failed to open output file for writing: " << out_path << std::endl;
  else
    std::cerr << "Wrote GPU BlockBPE tokens to " << out_path << std::endl;
  gtk_destroy(tok);
  return all_ok ? 0 : 1;
}
