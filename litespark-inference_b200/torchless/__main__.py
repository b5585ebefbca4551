"""Command line of the torchless runtime on the GPU backend.

    python litespark-inference_b200/torchless/__main__.py info
    python litespark-inference_b200/torchless/__main__.py generate "12 845 9" --model synthetic-toy --max-tokens 16
    python litespark-inference_b200/torchless/__main__.py benchmark --model synthetic-bitnet-2b --tokens 128
    python litespark-inference_b200/torchless/__main__.py chat --model /path/to/checkpoint

The four commands of the reference's CLI (litespark_inference/torchless/__main__.py:354-397: generate, info,
benchmark, chat) with the same flags, printing the same report lines.  ``benchmark --inference`` follows the
protocol of the reference's kernel benchmark (benchmark_kernel.py:814-876): one warm-up prefill, five timed
prefills of a 128-token prompt, three greedy tg passes, mean +- standard deviation.

Where the models come from: ``--model`` is a LOCAL checkpoint directory (``config.json`` + ``model.safetensors``,
optionally ``tokenizer.json``; BitNet master weights or a Falcon-E packed checkpoint, told apart by their
tensors), or one of the seeded random-init stand-ins ``synthetic-bitnet-2b`` / ``synthetic-toy`` /
``synthetic-falcon-toy``.  Nothing is downloaded.  Without a ``tokenizer.json`` the text side degrades to
space-separated token ids in, token ids out.
"""
from __future__ import annotations

import argparse
import platform
import statistics
import sys
import time
from pathlib import Path

if __package__ in (None, ""):
    # run as a script: register the hyphen-named source directory as the importable package
    import importlib.util
    _pkg_dir = Path(__file__).resolve().parent.parent
    _name = "litespark_inference_b200"
    if _name not in sys.modules:
        _spec = importlib.util.spec_from_file_location(_name, _pkg_dir / "__init__.py",
                                                       submodule_search_locations=[str(_pkg_dir)])
        _mod = importlib.util.module_from_spec(_spec)
        sys.modules[_name] = _mod
        _spec.loader.exec_module(_mod)
    __package__ = _name + ".torchless"

import numpy as np

SYNTHETIC = ("synthetic-bitnet-2b", "synthetic-toy", "synthetic-falcon-toy")
PROMPT_TEXT = "The quick brown fox jumps over the lazy dog."


def _kernel_label() -> str:
    return "sm100 (torchless, extern \"C\" CUDA: dp4a GEMV / mma.sync / tcgen05 GEMM)"


def load_model_and_tokenizer(name: str, embed_dtype: str):
    """(host model, tokenizer, is_falcon) for a checkpoint directory or a synthetic stand-in."""
    from . import loader, synthetic
    from .tokenizer import IdTokenizer, LocalTokenizer
    if name in SYNTHETIC:
        if name == "synthetic-falcon-toy":
            return synthetic.random_falcon_model(synthetic.toy_falcon_config(), seed=0), IdTokenizer(), True
        cfg = synthetic.bitnet_2b_config() if name == "synthetic-bitnet-2b" else synthetic.toy_config()
        return synthetic.random_model(cfg, seed=0, fast=True), IdTokenizer(), False
    d = Path(name)
    if not d.is_dir():
        raise ValueError(f"unknown model {name!r}: give a checkpoint directory or one of {', '.join(SYNTHETIC)} "
                         "(this build never downloads a checkpoint)")
    from .safetensors_io import open_safetensors
    sf = open_safetensors(d / "model.safetensors")
    falcon = sf.header["model.layers.0.self_attn.q_proj.weight"]["dtype"] == "U8"
    sf.close()
    model = loader.load_falcon_dir(d, embed_dtype=embed_dtype) if falcon else loader.load_bitnet_dir(d, embed_dtype=embed_dtype)
    tok = LocalTokenizer(d) if (d / "tokenizer.json").exists() else IdTokenizer()
    return model, tok, falcon


def _prompt_ids(tok, text: str, vocab: int, n: int = 0):
    """Token ids of `text`; with the id stand-in tokenizer a non-numeric text becomes seeded random ids."""
    try:
        ids = [int(t) for t in tok.encode(text)]
    except ValueError:
        ids = [int(t) for t in np.random.default_rng(len(text)).integers(0, vocab, max(n, len(text.split())))]
    if n:
        ids = (ids * (n // max(len(ids), 1) + 1))[:n]
    return [min(max(t, 0), vocab - 1) for t in ids]


def cmd_info(args) -> int:
    from . import kernel
    print("litespark_inference_b200.torchless")
    print(f"  platform : {platform.system()} {platform.machine()}")
    print(f"  python   : {platform.python_version()}")
    print(f"  kernel   : {kernel.library_path()}" + ("" if kernel.library_path().exists() else "  (not built)"))
    try:
        lib = kernel.load_library(True)
        print(f"  GPU      : device {lib.lspk_sm_count()} SMs, {_kernel_label()}")
        print(f"  OpenMP   : {kernel.has_omp()}  (max_threads={kernel.max_threads()})")
    except kernel.KernelUnavailable as ex:
        print(f"  GPU      : unavailable ({ex}); there is no CPU fallback")
    print(f"  Accelerate: {kernel.has_accelerate()}")
    return 0


def cmd_generate(args) -> int:
    from . import runtime as rt
    print("Loading tokenizer...", flush=True)
    t0 = time.perf_counter()
    model, tok, falcon = load_model_and_tokenizer(args.model, args.embed_dtype)
    dm = rt.to_device(model)
    print(f"  {time.perf_counter() - t0:.2f}s")
    text = args.prompt if args.raw else tok.format_chat(args.prompt)
    ids = _prompt_ids(tok, text, model.config.vocab_size)
    print(f"Prompt ({len(ids)} tokens): {text!r}", flush=True)
    state = rt.init_state(dm, t_max=len(ids) + args.max_tokens + 1)
    print("Prefill...", flush=True)
    t0 = time.perf_counter()
    logits = rt.forward_prefill(dm, state, ids)
    dt = time.perf_counter() - t0
    print(f"  {len(ids)} tokens in {dt:.2f}s ({len(ids) / dt:.2f} tok/s)")
    print("Generate:", flush=True)
    eos = set(getattr(model.config, "eos_token_ids", ()))
    eos.update(getattr(tok, "stop_token_ids", ()))
    generated, shown = [], ""
    t0 = time.perf_counter()
    for _ in range(args.max_tokens):
        nxt = int(np.argmax(logits))
        if nxt in eos and not args.ignore_eos:
            break
        generated.append(nxt)
        now = tok.decode(generated)
        if "\ufffd" not in now and now.startswith(shown):
            print(now[len(shown):], end="", flush=True)
            shown = now
        logits = rt.forward_one(dm, state, nxt)
    dt = time.perf_counter() - t0
    out = tok.decode(generated)
    if out.startswith(shown):
        print(out[len(shown):], end="", flush=True)
    print()
    if generated:
        print(f"\nGenerated {len(generated)} tokens in {dt:.2f}s ({len(generated) / dt:.2f} tok/s)")
    print("\n--- output ---")
    print(out)
    return 0


def cmd_benchmark(args) -> int:
    from . import kernel
    from . import runtime as rt
    print("Litespark-Inference Benchmark (torchless)")
    print("=" * 60)
    print(f"\nArchitecture: {platform.machine()}")
    print(f"Platform: {platform.system()}")
    print(f"Kernel: {_kernel_label()} (OMP={kernel.has_omp()} max_threads={kernel.max_threads()})")
    print(f"\nLoading model: {args.model} (embed_dtype={args.embed_dtype})")
    t0 = time.perf_counter()
    model, tok, falcon = load_model_and_tokenizer(args.model, args.embed_dtype)
    dm = rt.to_device(model)
    load_t = time.perf_counter() - t0
    MB = 1024 * 1024
    dev_mb = dm.device_bytes / MB
    print(f"Memory: {dev_mb:.0f} MB on the device")
    print(f"Load time: {load_t:.2f}s")
    V = model.config.vocab_size

    if args.inference:
        # the kernel benchmark's protocol: 128 prompt tokens, 1 warm-up, 5 x pp, 3 x tg, mean +- std
        ids = _prompt_ids(tok, (PROMPT_TEXT + " ") * 20, V, 128)
        t_max = len(ids) + args.tokens + 4
        print(f"Prompt tokens: {len(ids)}")
        print(f"Generate tokens: {args.tokens}")
        print("\nWarming up...")
        rt.forward_prefill(dm, rt.init_state(dm, t_max=t_max), ids)
        print("\nPrompt Processing (pp):")
        pp = []
        for _ in range(5):
            st = rt.init_state(dm, t_max=t_max)
            t0 = time.perf_counter()
            rt.forward_prefill(dm, st, ids)
            pp.append((time.perf_counter() - t0) * 1000)
        pp_mean = statistics.mean(pp)
        print(f"  Time: {pp_mean:.2f}±{statistics.stdev(pp):.2f} ms")
        print(f"  Throughput: {len(ids) / (pp_mean / 1000):.2f} tokens/sec")
        print(f"\nToken Generation (tg{args.tokens}):")
        tg = []
        for _ in range(3):
            st = rt.init_state(dm, t_max=t_max)
            logits = rt.forward_prefill(dm, st, ids)
            t0 = time.perf_counter()
            for _ in range(args.tokens):
                logits = rt.forward_one(dm, st, int(np.argmax(logits)))
            tg.append(time.perf_counter() - t0)
        tg_mean = statistics.mean(tg)
        print(f"  Time: {tg_mean * 1000:.2f}±{statistics.stdev(tg) * 1000:.2f} ms")
        print(f"  Throughput: {args.tokens / tg_mean:.2f} tokens/sec")
        # the same loop without the logits leaving the GPU (greedy choice made on the device)
        st = rt.init_state(dm, t_max=t_max)
        first = rt.prefill_first_token(st, ids)
        t0 = time.perf_counter()
        rt.decode_greedy(st, first, args.tokens + 1)
        dt = time.perf_counter() - t0
        print(f"  On-device greedy loop: {dt * 1000:.2f} ms ({args.tokens / dt:.2f} tokens/sec)")
        return 0

    ids = _prompt_ids(tok, PROMPT_TEXT, V)
    print(f"\nBenchmarking with prompt: '{PROMPT_TEXT}' ({len(ids)} tokens)")
    print("-" * 60)
    print("Warming up...", flush=True)
    for _ in range(3):
        rt.forward_prefill(dm, rt.init_state(dm, t_max=len(ids) + 1), ids)
    print("\nTime to First Token (TTFT):")
    times = []
    for _ in range(10):
        st = rt.init_state(dm, t_max=len(ids) + 1)
        t0 = time.perf_counter()
        rt.forward_prefill(dm, st, ids)
        times.append((time.perf_counter() - t0) * 1000)
    ttft = sum(times) / len(times)
    print(f"  Average: {ttft:.2f} ms")
    print(f"  Minimum: {min(times):.2f} ms")
    print(f"\nGeneration Speed ({args.tokens} tokens):")
    times = []
    for _ in range(3):
        st = rt.init_state(dm, t_max=len(ids) + args.tokens + 1)
        logits = rt.forward_prefill(dm, st, ids)
        t0 = time.perf_counter()
        for _ in range(args.tokens):
            logits = rt.forward_one(dm, st, int(np.argmax(logits)))
        times.append(time.perf_counter() - t0)
    gen = sum(times) / len(times)
    tps = args.tokens / gen
    print(f"  Average: {gen * 1000:.0f} ms ({tps:.2f} tokens/sec)")
    print("\n" + "=" * 60)
    print("SUMMARY")
    print("=" * 60)
    print(f"Model:      {args.model}")
    print(f"Backend:    torchless sm100 (embed_dtype={args.embed_dtype})")
    print(f"Memory:     {dev_mb:.0f} MB")
    print(f"TTFT:       {ttft:.2f} ms")
    print(f"Throughput: {tps:.2f} tokens/sec")
    return 0


def cmd_chat(args) -> int:
    from . import runtime as rt
    print("Loading tokenizer and model...", flush=True)
    model, tok, falcon = load_model_and_tokenizer(args.model, args.embed_dtype)
    dm = rt.to_device(model)
    print("\nLitespark-Inference Chat (torchless)")
    print("Type 'quit' or 'exit' to end the conversation")
    print("-" * 50)
    system = ("You are Litespark, a helpful AI assistant running locally. "
              "Provide accurate, concise, and practical answers.")
    users, answers = [], []
    eos = set(getattr(model.config, "eos_token_ids", ()))
    eos.update(getattr(tok, "stop_token_ids", ()))
    while True:
        try:
            line = input("\nYou: ").strip()
        except (EOFError, KeyboardInterrupt):
            print("\nGoodbye!")
            break
        if line.lower() in ("quit", "exit", "q"):
            print("Goodbye!")
            break
        if not line:
            continue
        users.append(line)
        pieces = [system, ""]
        for u, a in zip(users[:-1], answers):
            pieces += [f"Question: {u}", f"Answer: {a}"]
        pieces += [f"Question: {line}", "Answer:"]
        ids = _prompt_ids(tok, "\n".join(pieces) if hasattr(tok, "_tok") else line, model.config.vocab_size)
        st = rt.init_state(dm, t_max=len(ids) + args.max_tokens + 1)
        logits = rt.forward_prefill(dm, st, ids)
        print("\nAssistant: ", end="", flush=True)
        gen, shown = [], ""
        for _ in range(args.max_tokens):
            nxt = int(np.argmax(logits))
            if nxt in eos:
                break
            gen.append(nxt)
            now = tok.decode(gen)
            if "\ufffd" not in now and now.startswith(shown):
                print(now[len(shown):], end="", flush=True)
                shown = now
            logits = rt.forward_one(dm, st, nxt)
        reply = tok.decode(gen)
        if reply.startswith(shown):
            print(reply[len(shown):], end="", flush=True)
        print()
        answers.append(reply)
        st.close()
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="litespark_inference_b200.torchless")
    sub = p.add_subparsers(dest="cmd", required=True)
    pg = sub.add_parser("generate", help="Greedy-decode a continuation")
    pg.add_argument("prompt", type=str)
    pg.add_argument("--model", "-m", type=str, default="synthetic-bitnet-2b")
    pg.add_argument("--max-tokens", type=int, default=32)
    pg.add_argument("--embed-dtype", choices=["bf16", "int8", "int4"], default="int4")
    pg.add_argument("--raw", action="store_true", help="Skip the chat-format wrapper around the prompt.")
    pg.add_argument("--ignore-eos", action="store_true", help="Keep generating even after EOS is produced.")
    pg.set_defaults(func=cmd_generate)
    pi = sub.add_parser("info", help="Show build/runtime info")
    pi.set_defaults(func=cmd_info)
    pb = sub.add_parser("benchmark", help="Run a pp/tg mini benchmark")
    pb.add_argument("--model", type=str, default="synthetic-bitnet-2b")
    pb.add_argument("--tokens", type=int, default=32, help="Tokens to generate for the tg measurement.")
    pb.add_argument("--embed-dtype", choices=["bf16", "int8", "int4"], default="int4")
    pb.add_argument("--inference", action="store_true",
                    help="The kernel benchmark's protocol: pp128 five times, tg three times, mean and deviation.")
    pb.set_defaults(func=cmd_benchmark)
    pc = sub.add_parser("chat", help="Interactive chat (greedy decode)")
    pc.add_argument("--model", type=str, default="synthetic-bitnet-2b")
    pc.add_argument("--max-tokens", type=int, default=256)
    pc.add_argument("--embed-dtype", choices=["bf16", "int8", "int4"], default="int4")
    pc.set_defaults(func=cmd_chat)
    args = p.parse_args(argv)
    from . import kernel
    try:
        return args.func(args)
    except kernel.KernelUnavailable as ex:
        print(f"error: {ex} (there is no CPU fallback)", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
