"""Makes tests/golden/tiny_a_reference.safetensors + .json: the logits and the
greedy tokens that TheEpicDolphin/gllm's OWN model code (imported unmodified
from a checkout, on the CPU, in float32) gives on tiny model A with random
weights.  tests/test_plain.py compares the plain implementation with them.

    python tests/golden/make_golden.py /path/to/gllm-checkout

Only the hub download is replaced: ``gllm.model.model.hf_hub_download`` is bound
to a function that returns ``<folder>/<filename>``, so the reference reads a
local folder.  The folder gets what the reference insists on: ``head_dim``,
``torch_dtype`` and a list ``eos_token_id`` in config.json, and a word-level
``tokenizer.json`` in which the text "5 17 3" is the ids [5, 17, 3].
Logits come from the reference's own calls (gllm/llm/llm.py:145,321-335):
``prepare_batch`` -> ``get_token_embeddings`` -> ``forward`` -> ``compute_logits``.
"""

import json
import os
import sys
import tempfile

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def main(reference_root: str) -> None:
    from tiny_models import write_tiny

    sys.path.insert(0, reference_root)
    import gllm.model.model as ref_model
    from gllm.config.generator_params import GeneratorParams
    from gllm.engine.llm_engine import LLMEngine
    from gllm.engine.llm_engine_base import GenerationRequest
    from gllm.scheduler.request_state import RequestState
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    ref_model.hf_hub_download = lambda repo_id, filename, cache_dir=None: os.path.join(repo_id, filename)
    tmp = tempfile.mkdtemp()
    folder = write_tiny("A", os.path.join(tmp, "model"))
    tok = Tokenizer(WordLevel({str(i): i for i in range(256)}, unk_token="0"))
    tok.pre_tokenizer = WhitespaceSplit()
    tok.save(os.path.join(folder, "tokenizer.json"))

    params = GeneratorParams(block_size=4, max_batch_size=4, max_seq_len=32, model_dtype="float32", kv_dtype="float32")
    engine = LLMEngine(hf_model=folder, gen_params=params, device="cpu", local_cache_dir=os.path.join(tmp, "cache"))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 255, (n,), generator=g).tolist() for n in (5, 9, 13)]
    out, meta = {}, {"prompts": prompts, "greedy": []}
    for i, p in enumerate(prompts):
        state = RequestState(id=1000 + i, prompt_token_ids=p, generated_token_ids=[], generated_logprobs=[],
                             is_finished=False, max_new_tokens=1, stop_token_ids=set(), temperature=1.0, top_k=1,
                             top_p=1.0, max_num_logprobs=0, future=None)
        batch = engine.llm.prepare_batch([state])
        hidden = engine.llm.model.get_token_embeddings(batch.query_token_ids)
        hidden = engine.llm.model.forward(hidden, batch.positions, batch.attention_metadata)
        out[f"logits_{i}"] = engine.llm.model.compute_logits(hidden)[0].float().contiguous()
    for p in prompts:                       # one by one: the reference breaks when a non-last request leaves a batch
        req = GenerationRequest(prompt=" ".join(map(str, p)), max_new_tokens=8, stop_tokens=[], temperature=0.1,
                                top_k=1, top_p=1.0)
        meta["greedy"].append(engine.generate([req])[0].token_ids)
    save_file(out, os.path.join(HERE, "tiny_a_reference.safetensors"))
    with open(os.path.join(HERE, "tiny_a_reference.json"), "w") as f:
        json.dump(meta, f)
    print("wrote", sorted(out), meta["greedy"])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/gllm-checkout")
    main(sys.argv[1])
