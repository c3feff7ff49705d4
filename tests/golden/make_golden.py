"""Makes the files under tests/golden/: logits (and greedy tokens) that
TheEpicDolphin/gllm's OWN model code (imported unmodified from a checkout, on
the CPU, in float32) gives on the tiny models A and B with random weights.
tests/test_plain.py compares the plain implementation with them.

    python tests/golden/make_golden.py /path/to/gllm-checkout

Only the hub download is replaced: ``gllm.model.model.hf_hub_download`` is bound
to a function that returns ``<folder>/<filename>``, so the reference reads a
local folder.  The folder gets what the reference insists on: ``head_dim``,
``torch_dtype`` and a list ``eos_token_id`` in config.json, and a word-level
``tokenizer.json`` in which the text "5 17 3" is the ids [5, 17, 3].
Logits come from the reference's own calls (gllm/llm/llm.py:145,321-335):
``prepare_batch`` -> ``get_token_embeddings`` -> ``forward`` -> ``compute_logits``.

tiny_a_reference: (1) each of three prompts whole, every position; (2) greedy
continuations by ``generate()``; (3) one request decoded token by token through
the reference's cache (its tokens fixed beforehand); (4) requests that arrive
with their whole prompts beside neighbours that are decoding.  Nobody leaves a
batch before the last step: the reference breaks when a request that is not the
last of its list leaves (gllm/llm/llm.py:163-191).

tiny_b_reference: tiny B has two things the reference lacks.  Its llama3
frequency scaling enters by overwriting the engine's ``cos_pos_cache`` and
``sin_pos_cache`` (gllm/model/model.py:126-128) after construction with tables
made from the PLAIN implementation's frequencies; its untied head by putting
``lm_head.weight`` in the place of ``model.embedding`` for the ``compute_logits``
call (gllm/model/model.py:232-239).  So this file anchors everything of B (one
kv head for three query heads, head size 32, three layers, drawn norm weights,
eps 1e-6, widths that are multiples of no tile) except the scaling rule itself
and the choice of the head matrix, which rest on their published meaning.
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


def _folder(name, tmp, vocab):
    from tiny_models import write_tiny
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    folder = write_tiny(name, os.path.join(tmp, "model" + name))
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    if not isinstance(cfg["eos_token_id"], list):
        cfg["eos_token_id"] = [cfg["eos_token_id"]]
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
    tok = Tokenizer(WordLevel({str(i): i for i in range(vocab)}, unk_token="0"))
    tok.pre_tokenizer = WhitespaceSplit()
    tok.save(os.path.join(folder, "tokenizer.json"))
    return folder


def main(reference_root: str) -> None:
    from plain_llama import plain_inverse_frequencies
    from tiny_models import TINY_B, read_raw

    sys.path.insert(0, reference_root)
    import gllm.model.model as ref_model
    from gllm.config.generator_params import GeneratorParams
    from gllm.engine.llm_engine import LLMEngine
    from gllm.engine.llm_engine_base import GenerationRequest
    from gllm.scheduler.request_state import RequestState

    ref_model.hf_hub_download = lambda repo_id, filename, cache_dir=None: os.path.join(repo_id, filename)
    tmp = tempfile.mkdtemp()

    def state(rid, prompt):
        return RequestState(id=rid, prompt_token_ids=prompt, generated_token_ids=[], generated_logprobs=[],
                            is_finished=False, max_new_tokens=64, stop_token_ids=set(), temperature=1.0, top_k=1,
                            top_p=1.0, max_num_logprobs=0, future=None)

    def step_logits(engine, states, head=None):
        """Logits of every request's own query rows in one step of the reference:
        list of [query_len, vocab]."""
        model = engine.llm.model
        batch = engine.llm.prepare_batch(states)
        hidden = model.get_token_embeddings(batch.query_token_ids)
        hidden = model.forward(hidden, batch.positions, batch.attention_metadata)
        table = model.embedding
        if head is not None:
            model.embedding = head
        logits = model.compute_logits(hidden)
        model.embedding = table
        lens = batch.attention_metadata.query_lens.tolist()
        return [logits[i, :n].float().contiguous().clone() for i, n in enumerate(lens)]

    # ------------------------------------------------------------------ tiny A
    folder = _folder("A", tmp, 256)
    params = GeneratorParams(block_size=4, max_batch_size=4, max_seq_len=32, model_dtype="float32", kv_dtype="float32")

    def engine_a():
        return LLMEngine(hf_model=folder, gen_params=params, device="cpu", local_cache_dir=os.path.join(tmp, "cache"))

    engine = engine_a()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 255, (n,), generator=g).tolist() for n in (5, 9, 13)]
    continuations = [torch.randint(0, 255, (6,), generator=g).tolist() for _ in prompts]
    out, meta = {}, {"prompts": prompts, "greedy": [], "continuations": continuations}
    for i, p in enumerate(prompts):
        out[f"logits_{i}"] = step_logits(engine, [state(1000 + i, p)])[0]
    for p in prompts:                       # one by one: the reference breaks when a non-last request leaves a batch
        req = GenerationRequest(prompt=" ".join(map(str, p)), max_new_tokens=8, stop_tokens=[], temperature=0.1,
                                top_k=1, top_p=1.0)
        meta["greedy"].append(engine.generate([req])[0].token_ids)
    # (3) the longest prompt, then its fixed continuation token by token from the reference's cache
    engine = engine_a()
    st = state(1, prompts[2])
    step_logits(engine, [st])
    rows = []
    for t in continuations[2]:
        st.generated_token_ids.append(t)
        rows.append(step_logits(engine, [st])[0][0])
    out["decode_2"] = torch.stack(rows)
    # (4) arrivals beside decoding neighbours: [0], [0, 1], [0, 1, 2], [0, 1, 2]; continuation tokens fixed
    engine = engine_a()
    states = [state(10 + i, p) for i, p in enumerate(prompts)]
    fed = [0, 0, 0]
    meta["mixed_schedule"] = [[0], [0, 1], [0, 1, 2], [0, 1, 2]]
    for s, active in enumerate(meta["mixed_schedule"]):
        for i in active:
            if fed[i]:                                   # not its first step: it brings its next fixed token
                states[i].generated_token_ids.append(continuations[i][fed[i] - 1])
        got = step_logits(engine, [states[i] for i in active])
        for i, rows in zip(active, got):
            out[f"mixed_{s}_{i}"] = rows
            fed[i] += 1
    save_file(out, os.path.join(HERE, "tiny_a_reference.safetensors"))
    with open(os.path.join(HERE, "tiny_a_reference.json"), "w") as f:
        json.dump(meta, f)
    print("wrote A:", sorted(out), meta["greedy"])

    # ------------------------------------------------------------------ tiny B
    folder = _folder("B", tmp, 384)
    _, weights = read_raw(folder)
    params = GeneratorParams(block_size=8, max_batch_size=4, max_seq_len=64, model_dtype="float32", kv_dtype="float32")
    engine = LLMEngine(hf_model=folder, gen_params=params, device="cpu", local_cache_dir=os.path.join(tmp, "cacheB"))
    model = engine.llm.model
    inv_freq = plain_inverse_frequencies(dict(TINY_B)).to(torch.float32)
    angles = torch.arange(params.max_seq_len, dtype=torch.float32)[:, None] * inv_freq[None, :]
    assert model.cos_pos_cache.shape == angles.shape
    model.cos_pos_cache = torch.cos(angles)
    model.sin_pos_cache = torch.sin(angles)
    head = weights["lm_head.weight"].to(torch.float32)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 383, (n,), generator=g).tolist() for n in (1, 7, 16, 23, 40)]
    continuation = torch.randint(0, 383, (12,), generator=g).tolist()
    out, meta = {}, {"prompts": prompts, "continuation": continuation}
    for i, p in enumerate(prompts):
        out[f"logits_{i}"] = step_logits(engine, [state(2000 + i, p)], head=head)[0]
    # the 23-token prompt, then twelve fixed tokens one by one (crosses pages of 8 at 24 and 32)
    st = state(3000, prompts[3])
    step_logits(engine, [st], head=head)
    rows = []
    for t in continuation:
        st.generated_token_ids.append(t)
        rows.append(step_logits(engine, [st], head=head)[0][0])
    out["decode_3"] = torch.stack(rows)
    save_file(out, os.path.join(HERE, "tiny_b_reference.safetensors"))
    with open(os.path.join(HERE, "tiny_b_reference.json"), "w") as f:
        json.dump(meta, f)
    print("wrote B:", sorted(out))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/gllm-checkout")
    main(sys.argv[1])
