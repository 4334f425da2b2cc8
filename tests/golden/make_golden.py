"""Writes tests/golden/*.npz: logits of the reference's own model code for the tiny test configurations.

Run once on a CPU (no GPU, no network):  python tests/golden/make_golden.py /path/to/fusezap-core
It writes each tiny model folder with this package's random-weights mode into a temporary folder, loads that folder
with the reference's `load_model(dir, float32, "NPY")` (its numpy device) and stores, for one seeded prompt,
  logits       (T, V) float32 of `Llama.forward(..., last_only=False)` (fusezap/serve/models/llama.py:539-616)
  ids          the prompt
  engine_ids   greedy tokens of the reference's paged engine for two prompts (fusezap/serve/engine.py:750-763)
The sliding-window configuration is left out: the reference applies a window to `llama`/`qwen2` configs only through
`use_sliding_window` on every layer, while the test configuration mixes windowed and full layers.
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def main(ref_root: str) -> None:
    os.environ.setdefault("FZ_CACHE_DIR", tempfile.mkdtemp())
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    from fusezap.dtype import dtypes
    from fusezap.tensor import Tensor
    from fusezap.serve.models import load_model
    from fusezap.serve.engine import LLMEngine, SamplingParams
    from fusezap_core_b200.weights import write_random_model
    from tiny_configs import get
    for name, T in (("tiny_llama", 40), ("tiny_qwen2", 40)):
        cfg, o = get(name)
        d = tempfile.mkdtemp()
        write_random_model(cfg, d, o["seed"], "float32", o["norm_noise"], std_scale=4.0)
        m = load_model(d, dtype=dtypes.float32, device="NPY", max_len=64, prefill_chunk=16)
        ids = np.random.default_rng(1).integers(0, cfg["vocab_size"], T)
        x = Tensor(m.embed(ids[None]), device="NPY", dtype=dtypes.float32)
        lg = m.forward(x, m.cache, 0, T, last_only=False).numpy()[0]
        m.reset()
        eng = LLMEngine(m, num_blocks=16, block_size=o["page_size"], max_num_seqs=2, max_prefill_tokens=8,
                        max_model_len=64, decode_beam=0)
        out = eng.generate([ids[:11].tolist(), ids[20:25].tolist()], SamplingParams(max_tokens=6, ignore_eos=True))
        np.savez(os.path.join(HERE, f"{name}.npz"), logits=lg.astype(np.float32), ids=ids.astype(np.int64),
                 engine_ids=np.asarray(out, np.int64))
        print(name, lg.shape, float(np.abs(lg).max()), out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/fusezap-core")
    main(sys.argv[1])
