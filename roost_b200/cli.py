"""The ``roost`` command line.

The reference's command is ``roost serve`` (an HTTP server, not built here) and ``roost doctor``
(src/Starlings.Roost.Server/RoostCli.cs:60-80); its worker takes ``--model --weights --kernels --device
--max-tokens --max-sequences --attention-blocks --recurrent-slots``
(src/Starlings.Roost.WorkerHost/WorkerArguments.cs:14-26). The same names and meanings are kept where they
apply: ``--model`` names what to serve (here a folder with config.json and model.safetensors), ``--kernels`` a
folder holding the kernel library, ``--device`` the CUDA ordinal, ``--max-tokens`` and ``--max-sequences`` the
largest token and row count of a step, ``--attention-blocks`` the pages of each paged pool. Parsing is strict
in the reference's manner (:408-438): an unknown option, a missing value or a repeated option is a usage error
and exits with 2.

    roost generate --model DIR (--prompt-ids 1,2,3 | --prompt-file FILE) [--max-output-tokens N] [--temperature T]
                   [--top-p P] [--top-k K] [--min-p P] [--seed S] [--stop-ids a,b] [--ignore-eos] [--repetition-penalty R]
                   [--frequency-penalty F] [--presence-penalty P] [--logprobs] [--top-logprobs N] [engine options]
    roost chat --model DIR [--tokenizer tokenizer.json] [--template TEXT] [--stop-strings TEXT|JSON-LIST] [--max-output-tokens N]
               [sampling options as for generate] [engine options]  a console: /reset clears the conversation, /exit quits
    roost bench --model DIR [--batch N] [--prompt-tokens P] [--new-tokens K] [--seed S] [engine options]
                                                      prefill and decode tokens a second of this model, one JSON line
    roost random-weights --config config.json --out DIR [--seed S] [--std X] [--norm-std X] [--mode normal|reference]
                                                      reference: the reference's own seeded generator (its tiny model's seed
                                                      unless --seed is given), so that its pinned tokens can be reproduced
    roost replay --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (bin/trace_run)
    roost doctor [--model DIR] [--kernels DIR] [--no-gpu] [--min-free-memory-gib N]
  engine options: [--dtype bfloat16|float32] [--device N] [--kernels DIR] [--page-size N] [--attention-blocks N]
                  [--kv-fraction F] [--max-tokens N] [--max-sequences N] [--max-chunk-tokens N]
"""
from __future__ import annotations

import json
import os
import sys

USAGE = __doc__.split("\n\n", 2)[2]

_ENGINE_VALUED = {"--dtype", "--device", "--kernels", "--page-size", "--attention-blocks", "--kv-fraction", "--max-tokens",
                  "--max-sequences", "--max-chunk-tokens"}
_COMMANDS = {
    "generate": (_ENGINE_VALUED | {"--model", "--prompt-ids", "--prompt-file", "--max-output-tokens", "--temperature", "--top-p",
                                   "--top-k", "--min-p", "--seed", "--stop-ids", "--repetition-penalty", "--frequency-penalty",
                                   "--presence-penalty", "--top-logprobs"}, {"--ignore-eos", "--logprobs"}),
    "chat": (_ENGINE_VALUED | {"--model", "--tokenizer", "--template", "--stop-strings", "--max-output-tokens", "--temperature", "--top-p", "--top-k",
                               "--min-p", "--seed", "--stop-ids", "--repetition-penalty", "--frequency-penalty", "--presence-penalty"},
             {"--ignore-eos"}),
    "bench": (_ENGINE_VALUED | {"--model", "--batch", "--prompt-tokens", "--new-tokens", "--seed"}, set()),
    "random-weights": ({"--config", "--out", "--seed", "--std", "--norm-std", "--mode"}, set()),
    "replay": ({"--model", "--dtype", "--out", "--max-tokens", "--page-size"}, set()),
    "doctor": ({"--model", "--kernels", "--min-free-memory-gib"}, {"--no-gpu"}),
}


class UsageError(Exception):
    pass


def parse(argv: list[str]) -> tuple[str, dict]:
    if not argv:
        raise UsageError("a command is needed")
    command, rest = argv[0], argv[1:]
    if command not in _COMMANDS:
        raise UsageError(f"unknown command '{command}'")
    valued, flags = _COMMANDS[command]
    out: dict = {}
    i = 0
    while i < len(rest):
        a = rest[i]
        if a in out:
            raise UsageError(f"option {a} is given twice")
        if a in flags:
            out[a] = True
            i += 1
        elif a in valued:
            if i + 1 >= len(rest):
                raise UsageError(f"option {a} needs a value")
            out[a] = rest[i + 1]
            i += 2
        else:
            raise UsageError(f"unknown option '{a}' for '{command}'")
    return command, out


def _int(opts, key, default=None):
    if key not in opts:
        return default
    try:
        return int(opts[key])
    except ValueError:
        raise UsageError(f"option {key} needs an integer, got '{opts[key]}'") from None


def _float(opts, key, default=None):
    if key not in opts:
        return default
    try:
        return float(opts[key])
    except ValueError:
        raise UsageError(f"option {key} needs a number, got '{opts[key]}'") from None


def _ids(text: str, key: str) -> list[int]:
    try:
        return [int(x) for x in text.replace(",", " ").split()]
    except ValueError:
        raise UsageError(f"option {key} needs token ids separated by commas or spaces") from None


def _need(opts, key):
    if key not in opts:
        raise UsageError(f"option {key} is required")
    return opts[key]


def _kv_fraction(opts) -> float:
    """--kv-fraction: the share of the device memory free after the weights that the cache pools take when
    --attention-blocks does not size them."""
    f = _float(opts, "--kv-fraction", 0.9)
    if not 0 < f <= 1:
        raise UsageError("--kv-fraction must lie in (0, 1]")
    return f


def _stop_strings(opts) -> tuple:
    """--stop-strings: one string, or a JSON list of strings."""
    if "--stop-strings" not in opts:
        return ()
    text = opts["--stop-strings"]
    if text.lstrip().startswith("["):
        try:
            stops = json.loads(text)
        except json.JSONDecodeError:
            raise UsageError("--stop-strings: not a JSON list") from None
    else:
        stops = [text]
    if not isinstance(stops, list) or not all(isinstance(x, str) and x for x in stops):
        raise UsageError("--stop-strings needs non-empty strings")
    return tuple(stops)


def _apply_common(opts) -> None:
    if "--device" in opts:
        os.environ["CUDA_VISIBLE_DEVICES"] = str(_int(opts, "--device"))
    if "--kernels" in opts:
        os.environ["ROOST_KERNELS"] = opts["--kernels"]


def cmd_generate(opts) -> int:
    model = _need(opts, "--model")
    if ("--prompt-ids" in opts) == ("--prompt-file" in opts):
        raise UsageError("exactly one of --prompt-ids and --prompt-file is needed")
    if "--prompt-ids" in opts:
        prompts = [_ids(opts["--prompt-ids"], "--prompt-ids")]
    else:
        with open(opts["--prompt-file"]) as f:
            prompts = [_ids(line, "--prompt-file") for line in f if line.strip()]
    if not prompts or any(not p for p in prompts):
        raise UsageError("a prompt is empty")
    dtype = opts.get("--dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise UsageError("--dtype is bfloat16 or float32")
    # every option is read before anything is loaded, so a bad value is a usage error whatever the model is
    engine_opts = dict(page_size=_int(opts, "--page-size", 16), attention_blocks=_int(opts, "--attention-blocks"), kv_fraction=_kv_fraction(opts),
                       max_sequences=_int(opts, "--max-sequences", 64), max_tokens=_int(opts, "--max-tokens", 2048),
                       max_chunk_tokens=_int(opts, "--max-chunk-tokens"))
    gen_opts = dict(max_output_tokens=_int(opts, "--max-output-tokens", 16), temperature=_float(opts, "--temperature"),
                    top_p=_float(opts, "--top-p"), top_k=_int(opts, "--top-k"), min_p=_float(opts, "--min-p"),
                    seed=_int(opts, "--seed"), stop_token_ids=tuple(_ids(opts.get("--stop-ids", ""), "--stop-ids")),
                    ignore_eos="--ignore-eos" in opts, repetition_penalty=_float(opts, "--repetition-penalty"),
                    frequency_penalty=_float(opts, "--frequency-penalty"), presence_penalty=_float(opts, "--presence-penalty"),
                    logprobs="--logprobs" in opts, top_logprobs=_int(opts, "--top-logprobs", 0))
    _check_sampling(gen_opts)
    _apply_common(opts)
    from .engine.engine import GenerationOptions, RoostEngine
    engine = RoostEngine(model, dtype=dtype, **engine_opts)
    go = GenerationOptions(**gen_opts)
    for prompt, out in zip(prompts, engine.generate(prompts, go)):
        line = {"prompt_tokens": len(prompt), "token_ids": out.token_ids, "finish_reason": out.finish_reason}
        if out.logprobs is not None:
            line["logprobs"] = out.logprobs
        if out.top_logprobs is not None:
            line["top_logprobs"] = [[[t, lp] for t, lp in alts] for alts in out.top_logprobs]
        print(json.dumps(line))
    return 0


def _check_sampling(gen_opts: dict) -> None:
    """The options' ranges, before anything is loaded: a bad value is a usage error."""
    from .engine.engine import GenerationOptions
    from .engine.request import RequestError
    try:
        GenerationOptions(**gen_opts).sampling().validate()
    except RequestError as e:
        raise UsageError(str(e)) from None


CHAT_TEMPLATE = "<|im_start|>user\n{message}<|im_end|>\n<|im_start|>assistant\n"


def cmd_chat(opts, lines=None, out=None) -> int:
    """A console in the manner of the reference's sample (samples/ChatConsole/Program.cs:84-120): a line is a turn,
    the whole conversation so far is the prompt of every turn, ``/reset`` clears it, ``/exit`` or an empty line
    quits; a turn that no longer fits is dropped with its error's code. With a tokenizer (``--tokenizer``, or
    tokenizer.json in the model folder, and the ``tokenizers`` package) a line is text, wrapped by ``--template``
    (``{message}`` is the line; the default is the ChatML turn Qwen3 checkpoints are tuned on) and the reply is printed
    as text; without one a line is token ids and so is the reply."""
    model = _need(opts, "--model")
    dtype = opts.get("--dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise UsageError("--dtype is bfloat16 or float32")
    engine_opts = dict(page_size=_int(opts, "--page-size", 16), attention_blocks=_int(opts, "--attention-blocks"), kv_fraction=_kv_fraction(opts),
                       max_sequences=_int(opts, "--max-sequences", 1), max_tokens=_int(opts, "--max-tokens", 2048),
                       max_chunk_tokens=_int(opts, "--max-chunk-tokens"))
    gen_opts = dict(max_output_tokens=_int(opts, "--max-output-tokens", 256), temperature=_float(opts, "--temperature"),
                    top_p=_float(opts, "--top-p"), top_k=_int(opts, "--top-k"), min_p=_float(opts, "--min-p"),
                    seed=_int(opts, "--seed"), stop_token_ids=tuple(_ids(opts.get("--stop-ids", ""), "--stop-ids")),
                    ignore_eos="--ignore-eos" in opts, repetition_penalty=_float(opts, "--repetition-penalty"),
                    frequency_penalty=_float(opts, "--frequency-penalty"), presence_penalty=_float(opts, "--presence-penalty"))
    _check_sampling(gen_opts)
    template = opts.get("--template", CHAT_TEMPLATE)
    if "{message}" not in template:
        raise UsageError("--template needs the placeholder {message}")
    stops = _stop_strings(opts)
    tokenizer_path = opts.get("--tokenizer") or os.path.join(model, "tokenizer.json")
    tokenizer = None
    if os.path.exists(tokenizer_path):
        try:
            from tokenizers import Tokenizer
        except ImportError:
            raise UsageError("a tokenizer file is given but the 'tokenizers' package is not installed") from None
        tokenizer = Tokenizer.from_file(tokenizer_path)
    elif "--tokenizer" in opts:
        raise UsageError(f"--tokenizer: {tokenizer_path} does not exist")
    if stops and tokenizer is None:
        raise UsageError("--stop-strings are matched on text: a tokenizer is needed")
    _apply_common(opts)
    from .engine.engine import GenerationOptions, RoostEngine
    from .engine.request import RequestError
    from .engine.text import IncrementalDetokenizer, StopMatcher
    out = out or sys.stdout
    engine = RoostEngine(model, dtype=dtype, **engine_opts)
    go = GenerationOptions(**gen_opts)
    print(f"Ready: {model}, {'text' if tokenizer else 'token ids'} in and out. /reset clears the conversation, /exit quits.", file=out, flush=True)
    history: list[int] = []
    lines = sys.stdin if lines is None else lines
    read = lines.readline if hasattr(lines, "readline") else (lambda it=iter(lines): next(it, ""))
    while True:
        print("> ", end="", file=out, flush=True)
        text = read().strip()
        if not text or text == "/exit":
            return 0
        if text == "/reset":
            history.clear()
            print("(conversation cleared)", file=out, flush=True)
            continue
        if tokenizer is not None:
            # turns are separated by a line break, as the template ends its own lines
            turn = tokenizer.encode(("\n" if history else "") + template.replace("{message}", text), add_special_tokens=False).ids
        else:
            try:
                turn = _ids(text, "a turn")
            except UsageError:
                print("[InvalidOption] a turn is token ids separated by commas or spaces", file=out, flush=True)
                continue
        reply: list[int] = []
        # text mode: the reply is detokenised as it grows (a token may end inside a character) and watched for the stop
        # strings, which end the turn and are not printed (src/Starlings.Generation.Roost/RoostChatClient.cs:366-378)
        detok = IncrementalDetokenizer(tokenizer, skip_special_tokens=True) if tokenizer is not None else None
        matcher = StopMatcher(stops)
        try:
            stream = engine.stream_completion(history + turn, go)
            for update in stream:
                if update.token is None:
                    continue
                reply.append(update.token)
                if tokenizer is None:
                    print(("" if len(reply) == 1 else " ") + str(update.token), end="", file=out, flush=True)
                    continue
                emit, matched = matcher.push(detok.push(update.token))
                print(emit, end="", file=out, flush=True)
                if matched is not None:
                    stream.close()     # cancels the request
                    break
            else:
                if tokenizer is not None:
                    emit, _ = matcher.push(detok.flush())
                    print(emit + matcher.flush(), end="", file=out, flush=True)
        except RequestError as e:
            print(f"\n[{e.kind}] {e} (type /reset to start over)", file=out, flush=True)
            continue
        print(file=out, flush=True)
        history += turn + reply


def cmd_bench(opts) -> int:
    """Times this model through the entry point: ``--batch`` requests of ``--prompt-tokens`` seeded random tokens each
    are prefilled (under the step's token budget) and then decode ``--new-tokens`` greedy tokens each. The first pass
    warms up (library handles, captured steps); the second is timed by wall clock with the device drained at both ends."""
    import random
    import time
    model = _need(opts, "--model")
    dtype = opts.get("--dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise UsageError("--dtype is bfloat16 or float32")
    batch, prompt_tokens, new_tokens = _int(opts, "--batch", 8), _int(opts, "--prompt-tokens", 512), _int(opts, "--new-tokens", 64)
    if min(batch, prompt_tokens, new_tokens) <= 0:
        raise UsageError("--batch, --prompt-tokens and --new-tokens must be positive")
    engine_opts = dict(page_size=_int(opts, "--page-size", 16), attention_blocks=_int(opts, "--attention-blocks"), kv_fraction=_kv_fraction(opts),
                       max_sequences=_int(opts, "--max-sequences", max(batch, 1)), max_tokens=_int(opts, "--max-tokens", 2048),
                       max_chunk_tokens=_int(opts, "--max-chunk-tokens"))
    seed = _int(opts, "--seed", 0)
    _apply_common(opts)
    import torch

    from .engine.engine import GenerationOptions, RoostEngine
    engine = RoostEngine(model, dtype=dtype, **engine_opts)
    rng = random.Random(seed)
    vocab = engine.model.spec.vocab
    prompts = [[rng.randrange(vocab) for _ in range(prompt_tokens)] for _ in range(batch)]
    sampling = GenerationOptions(max_output_tokens=new_tokens, ignore_eos=True).sampling()
    result = {}
    for timed in (False, True):
        for p in prompts:
            engine.add_request(p, sampling)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while any(s.generated == 0 for s in engine.scheduler.sequences()):     # until every request has its first token
            engine.step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        produced = 0
        while engine.has_unfinished():
            produced += sum(1 for e in engine.step() if e.token is not None)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        if timed:
            result = {"model": str(model), "dtype": dtype, "batch": batch, "prompt_tokens": prompt_tokens, "new_tokens": new_tokens,
                      "prefill_tokens_per_s": round(batch * prompt_tokens / (t1 - t0), 1), "prefill_s": round(t1 - t0, 4),
                      "decode_tokens_per_s": round(produced / (t2 - t1), 1) if t2 > t1 and produced else None,
                      "decode_ms_per_step": round((t2 - t1) / max(new_tokens - 1, 1) * 1e3, 3), **engine.stats()}
    print(json.dumps(result))
    return 0


def cmd_random_weights(opts) -> int:
    from .weights.random_init import REFERENCE_TINY_SEED, write_random_model
    mode = opts.get("--mode", "normal")
    if mode not in ("normal", "reference"):
        raise UsageError("--mode is normal or reference")
    if mode == "reference" and ("--std" in opts or "--norm-std" in opts):
        raise UsageError("--std and --norm-std do not apply to --mode reference: the reference's generator fixes the amplitudes")
    with open(_need(opts, "--config")) as f:
        config = json.load(f)
    seed = _int(opts, "--seed", REFERENCE_TINY_SEED if mode == "reference" else 0)
    out = write_random_model(_need(opts, "--out"), config, seed, _float(opts, "--std", 0.02), _float(opts, "--norm-std", 0.0), mode=mode)
    print(out)
    return 0


def cmd_replay(opts) -> int:
    from .replay import main
    args = []
    for k, v in opts.items():
        args += [k, v]
    return main(args)


def cmd_doctor(opts) -> int:
    """One line per check; exit 1 when a check fails (src/Starlings.Roost.Server/RoostCli.cs:76-80)."""
    _apply_common(opts)
    ok = True

    def line(name, good, detail):
        nonlocal ok
        ok = ok and good
        print(f"{'ok  ' if good else 'FAIL'} {name}: {detail}")

    from .kernels import build
    try:
        line("nvcc", True, build.find_nvcc())
    except build.BuildError as e:
        line("nvcc", False, str(e))
    try:
        line("kernel library", True, str(build.library_path()))
    except Exception as e:  # noqa: BLE001
        line("kernel library", False, str(e).splitlines()[0])
    if "--no-gpu" not in opts:
        import torch
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability()
            line("gpu", major == 10, f"{torch.cuda.get_device_name()} (sm_{major}{minor}); the library is built for sm_100a")
            free, total = torch.cuda.mem_get_info()
            want = _float(opts, "--min-free-memory-gib", 1.0)
            line("device memory", free / 2**30 >= want, f"{free / 2**30:.1f} GiB free of {total / 2**30:.1f}")
            try:
                from .kernels import library
                line("kernel ABI", True, f"version {library.load()._lib.roost_abi_version()}")
            except Exception as e:  # noqa: BLE001
                line("kernel ABI", False, str(e))
        else:
            line("gpu", False, "no CUDA device is visible")
    if "--model" in opts:
        try:
            from .engine.model import parameter_declarations, read_model_config
            from .weights import loader
            from .weights.safetensors_io import SafetensorsFile
            arch, cfg, _ = read_model_config(opts["--model"])
            line("config.json", True, f"{arch.name}")
            for w in getattr(cfg, "warnings", []):
                print(f"note config.json: {w}")
            tied = cfg.tie_word_embeddings
            if tied is None:
                tied = not loader.checkpoint_has(opts["--model"], "lm_head.weight")
            spec = arch.to_spec(cfg, tied)
            want = loader.expected_tensors(parameter_declarations(spec), spec.weight_names)
            have = {}
            weight_map = loader.checkpoint_index(opts["--model"])
            for f in loader.checkpoint_files(opts["--model"]):
                with SafetensorsFile(f) as st:
                    have.update({n: tuple(e.shape) for n, e in st.entries.items() if weight_map is None or weight_map.get(n) == f.name})
            missing = [n for n in want if n not in have]
            wrong = [n for n in want if n in have and have[n] != want[n]]
            line("weights", not missing and not wrong, f"{len(want)} tensors wanted, {len(missing)} missing, {len(wrong)} of another shape")
        except Exception as e:  # noqa: BLE001
            line("model", False, str(e).splitlines()[0])
    return 0 if ok else 1


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        command, opts = parse(argv)
        return {"generate": cmd_generate, "chat": cmd_chat, "bench": cmd_bench, "random-weights": cmd_random_weights, "replay": cmd_replay, "doctor": cmd_doctor}[command](opts)
    except UsageError as e:
        print(f"roost: {e}\n\nusage:\n{USAGE}", file=sys.stderr)
        return 2
    except (ValueError, RuntimeError, OSError) as e:  # a config, weight, request or kernel error: one line, no traceback
        print(f"roost: error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
