"""Child process of tests/test_gpu_vllm_e2e.py: builds a small random-init Llama checkpoint
(deterministic, N(0, 0.02) weights), runs it through `vllm.LLM` with either this repository's
attention backend (registered as CUSTOM, the enum member the reference plugin registers) or
vLLM's stock backend, and writes greedy tokens and log-probabilities to a JSON file.

    python tiny_llama_worker.py --prepare --workdir DIR          (writes the checkpoint, once)
    python tiny_llama_worker.py --backend custom|stock --out result.json --workdir DIR

The checkpoint is written by a process of its own: vLLM forks its engine process, and a fork
after this process has run multi-threaded CPU kernels (the weight initialisation) leaves the
child with a dead thread pool.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
PKG = os.path.join(ROOT, "tt-xla_b200")

TINY = dict(hidden_size=1024, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=8,
            num_key_value_heads=2, head_dim=128, vocab_size=2048, rope_theta=500000.0,
            max_position_embeddings=2048, rms_norm_eps=1e-5, tie_word_embeddings=False,
            hidden_act="silu", bos_token_id=1, eos_token_id=2)
PROMPT_LENS = (5, 70, 200, 600)      # the last one is prefilled in chunks (256-token step budget)
GEN_TOKENS = 12


def make_checkpoint(path: str) -> None:
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    if os.path.exists(os.path.join(path, "config.json")):
        return
    torch.manual_seed(1234)
    model = LlamaForCausalLM(LlamaConfig(**TINY)).to(torch.bfloat16)
    model.save_pretrained(path, safe_serialization=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", choices=["custom", "stock"])
    ap.add_argument("--out")
    ap.add_argument("--workdir", required=True)
    ap.add_argument("--kv-cache-dtype", default="auto")
    ap.add_argument("--prepare", action="store_true")
    args = ap.parse_args()
    model_dir = os.path.join(args.workdir, "tiny_llama")
    if args.prepare:
        make_checkpoint(model_dir)
        return
    assert args.backend and args.out, "--backend and --out are required"
    assert os.path.exists(os.path.join(model_dir, "config.json")), "run with --prepare first"

    # engine-core child processes find the plugin's entry point through PYTHONPATH
    os.environ["PYTHONPATH"] = PKG + os.pathsep + os.environ.get("PYTHONPATH", "")
    os.environ["B200ATTN_FUSED_ROW_PARALLEL"] = "0"
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    sys.path.insert(0, PKG)
    import torch
    from vllm import LLM, SamplingParams

    kw = dict(model=model_dir, skip_tokenizer_init=True, dtype="bfloat16", block_size=64,
              max_model_len=1024, max_num_seqs=8, max_num_batched_tokens=256,
              enable_chunked_prefill=True, gpu_memory_utilization=0.25, seed=0,
              enable_prefix_caching=False, kv_cache_dtype=args.kv_cache_dtype,
              compilation_config={"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY"})
    if args.backend == "custom":
        kw["attention_backend"] = "CUSTOM"
    llm = LLM(**kw)
    g = torch.Generator().manual_seed(7)
    prompts = [dict(prompt_token_ids=torch.randint(3, TINY["vocab_size"], (n,), generator=g).tolist())
               for n in PROMPT_LENS]
    sp = SamplingParams(max_tokens=GEN_TOKENS, temperature=0.0, ignore_eos=True, detokenize=False,
                        logprobs=5, prompt_logprobs=0)
    outs = llm.generate(prompts, sp, use_tqdm=False)
    result = []
    for p, o in zip(prompts, outs):
        ids = p["prompt_token_ids"]
        # log-probability of every prompt token given its prefix (position 0 has none)
        plp = [float(d[t].logprob) for t, d in zip(ids[1:], o.prompt_logprobs[1:])]
        c = o.outputs[0]
        steps = [{str(t): float(lp.logprob) for t, lp in d.items()} for d in c.logprobs]
        result.append({"tokens": list(c.token_ids), "prompt_logprobs": plp, "steps": steps})
    with open(args.out, "w") as f:
        json.dump({"backend": args.backend, "results": result}, f)
    try:
        llm.llm_engine.engine_core.shutdown()
    except Exception:
        pass
    # the result is on disk: leave without waiting for the engine's helper threads
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
