"""Makes the golden files of this folder from the two pieces of the upstream project
that run on a CPU.  Run once, by hand, with the upstream checkout at hand:

    python tests/golden/make_golden.py /path/to/kv_cache_optimization_for_llm

1. ``sampling_golden.json``: upstream's numpy mirror of its sampler
   (python/sampling_reference.py): ``counter_uniform`` on a grid of
   (seed, key, step), and the token picked by its one-level CDF (``flat_sample``)
   and by its two-level walk (``kernel_sample``) for given logits and draws.
2. ``rope_golden.json``: the host half of ``initRopeFrequencies``
   (base/src/kernels.cu:56-106) compiled with nvcc and run on the CPU, its two
   device calls redirected to host buffers; cos and sin rows of a few positions at
   the constants of base/src/config.h (head_dim 64, theta 500000, llama3 scaling
   32 / 1 / 4 / 8192).

The tests only read the JSON files; nothing at test time needs the upstream tree.
The rest of the upstream model code cannot be run without a GPU; what its whole engine
generates on one is recorded by ``make_upstream_tokens.py`` beside this file.
"""

import importlib.util
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

ROPE_MAIN = r'''
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>
#include "kernels.cuh"
static cudaError_t fake_malloc(float **p, size_t n) { *p = (float *)malloc(n); return cudaSuccess; }
static cudaError_t fake_memcpy(void *d, const void *s, size_t n, cudaMemcpyKind) { memcpy(d, s, n); return cudaSuccess; }
#define cudaMalloc(p, n) fake_malloc(p, n)
#define cudaMemcpy(d, s, n, k) fake_memcpy(d, s, n, k)
#include "kernels.cu"
int main() {
  initRopeFrequencies();
  const int positions[] = {0, 1, 2, 7, 100, 1023, 2047};
  printf("{\"head_dim\": %d, \"theta\": %.1f, \"factor\": %.1f, \"low_freq_factor\": %.1f, \"high_freq_factor\": %.1f, "
         "\"original_max_position_embeddings\": %d, \"rows\": {", HEAD_DIM, (double)ROPE_THETA,
         (double)ROPE_SCALING_FACTOR, (double)ROPE_LOW_FREQ_FACTOR, (double)ROPE_HIGH_FREQ_FACTOR, (int)ROPE_ORIGINAL_MAX_LEN);
  for (int k = 0; k < 7; ++k) {
    int pos = positions[k];
    printf("%s\"%d\": {\"cos\": [", k ? ", " : "", pos);
    for (int i = 0; i < HEAD_DIM / 2; ++i) printf("%s%.9g", i ? "," : "", d_cos_table[pos * HEAD_DIM + 2 * i]);
    printf("], \"sin\": [");
    for (int i = 0; i < HEAD_DIM / 2; ++i) printf("%s%.9g", i ? "," : "", d_sin_table[pos * HEAD_DIM + 2 * i]);
    printf("]}");
  }
  printf("}}\n");
  return 0;
}
'''


def sampling(upstream):
    spec = importlib.util.spec_from_file_location("sampling_reference", os.path.join(upstream, "python", "sampling_reference.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    uniforms = [[s, k, p, ref.counter_uniform(s, k, p)]
                for s in (0, 1, 99, 1234, 2**32 - 1) for k in (0, 7, 8 * 31 + 3, 2**31) for p in (0, 1, 512, 65535)]
    rng = np.random.default_rng(0)
    # the two-level walk is tied to upstream's vocabulary size, so its cases use that size
    logits = rng.normal(0.0, 2.0, ref.VOCAB_SIZE)
    logits[rng.choice(ref.VOCAB_SIZE, 20, replace=False)] += 12.0
    picks = []
    for temperature in (0.7, 1.0, 1.5):
        for i in range(40):
            u = ref.counter_uniform(1234, 7, i)
            flat = ref.flat_sample(logits, 1.0 / temperature, u)
            walk = ref.kernel_sample(logits, 1.0 / temperature, u)
            picks.append([temperature, i, u, int(flat), int(walk)])
    small = rng.normal(0.0, 1.5, 300)
    small_picks = [[t, i, int(ref.flat_sample(small, 1.0 / t, ref.counter_uniform(5, 2, i)))]
                   for t in (0.5, 1.0) for i in range(60)]
    out = {"uniform": uniforms, "big_logits_seed": 0, "big_picks": picks,
           "small_logits": small.tolist(), "small_picks": small_picks}
    json.dump(out, open(os.path.join(HERE, "sampling_golden.json"), "w"))


def rope(upstream):
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "rope_host.cu")
        open(src, "w").write(ROPE_MAIN)
        exe = os.path.join(d, "rope_host")
        subprocess.run(["nvcc", "-w", "-I", os.path.join(upstream, "base", "src"), "-I",
                        os.path.join(upstream, "base", "include"), "-o", exe, src], check=True)
        text = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    json.loads(text)
    open(os.path.join(HERE, "rope_golden.json"), "w").write(text)


if __name__ == "__main__":
    sampling(sys.argv[1])
    rope(sys.argv[1])
