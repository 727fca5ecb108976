#!/usr/bin/env bash
# Block-size x chunk-length sweep of the one-CTA-per-chunk kernel, with the CSV columns of the reference's
# profile_blockbpe_block_sizes.sh.  The reference rebuilds its binary per block size (-DBLOCK_SIZE); here the
# block size is a run-time setting of the same binary (GTK_BLOCK_SIZE).
#   usage: profile_blockbpe_block_sizes.sh [input_path]     (run from a directory that holds
#          data/gpt2_tokenizer/merges.txt, or set GTK_MERGES; GTK_OUTPUT picks the token file)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
input="${1:-data/input/pride_and_prejudice.txt}"
[[ -f "${input}" ]] || { echo "ERROR: Input file '${input}' not found." >&2; exit 1; }
echo "BlockBPE block-size profiling on '${input}'"
echo
echo "block_size,seq_len,cpu_ms,gpu_ms,gpu_tokens_per_s"
for bs in 128 256 512 1024; do
  for seq_len in 128 256 512 1024 2048 4096; do
    out="$(GTK_BLOCK_SIZE=${bs} "${here}/gpu_tokenizer_blockbpe" "${seq_len}" "${input}" base)"
    cpu_ms="$(grep 'CPU BPE (greedy Algorithm 1) time' <<< "${out}" | awk '{print $(NF-1)}')"
    gpu_ms="$(grep 'GPU BlockBPE-style greedy kernel time' <<< "${out}" | awk '{print $(NF-1)}')"
    tokps="$(grep 'GPU greedy kernel throughput:' <<< "${out}" | awk '{print $(NF-1)}')"
    echo "${bs},${seq_len},${cpu_ms},${gpu_ms},${tokps}"
  done
done
