"""``oxidize`` command line: run / chat / serve / pull / show / list / inspect / bench / gpu-cluster.

Ollama-style verbs are rewritten into flags before parsing, as the reference does
(``oxidize-cli/src/main/command_rewrite.rs:8``; flag surface ``oxidize-cli/src/main.rs:74-209`` and
``oxidize-server/src/cli.rs:72-160``).  Flag names and defaults are kept; ``--tp``, ``--pp``,
``--kv-page-size``, ``--max-running``, ``--max-batched-tokens``, ``--fused-comm`` and ``--tokens``
are additions.  ``--backend`` accepts the reference's values but only ``cpu`` and ``cuda`` run.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional

VERBS = ("run", "chat", "serve", "pull", "show", "list", "inspect", "bench", "gpu-cluster")
DEAD_BACKENDS = ("metal", "mlx", "rocm", "vulkan", "intel-arc")
MODEL_DIR = os.path.expanduser(os.environ.get("OXIDIZE_MODEL_DIR", "~/.cache/oxidize/models"))


def rewrite_args(argv: List[str]) -> List[str]:
    """``run M "prompt"`` → ``--model M --prompt "prompt"``; ``serve M`` → ``--model M --api-only`` …"""
    if not argv or argv[0] not in VERBS:
        return argv
    verb, rest = argv[0], argv[1:]
    pos = []
    flags = []
    i = 0
    while i < len(rest):
        a = rest[i]
        if a.startswith("-"):
            flags.append(a)
            if "=" not in a and i + 1 < len(rest) and not rest[i + 1].startswith("-") and a not in _BOOL_FLAGS:
                flags.append(rest[i + 1])
                i += 1
        else:
            pos.append(a)
        i += 1
    out = ["--verb", verb]
    if pos:
        out += ["--model", pos[0]]
    if verb == "run" and len(pos) > 1:
        out += ["--prompt", " ".join(pos[1:])]
    if verb == "chat":
        out += ["--chat"]
    if verb == "serve":
        out += ["--api-only"]
    return out + flags


_BOOL_FLAGS = {"--chat", "--cpu-optimized", "--ram-offload", "--mmap-prefetch", "--mmap-hugepages", "--layer-wise",
               "--turboquant-kv", "--no-turboquant-kv", "--mesh", "--auto", "--no-auto", "--no-api", "--serve-api",
               "--api-only", "--vision", "--force-dflash", "--no-mtp", "--quantspec", "--pipe-head", "--pipe-tail",
               "--turboquant", "--no-turboquant", "--json", "--bench-no-eos", "--cuda-graphs", "--no-cuda-graphs"}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="oxidize", description="Blackwell-native LLM inference engine")
    a = p.add_argument
    a("--verb", default="run", choices=VERBS, help=argparse.SUPPRESS)
    a("--model", default=None)
    a("--prompt", default="hello")
    a("--tokens", default=None, help="raw token-id prompt, e.g. 1,2,3")
    a("--chat", action="store_true")
    a("--backend", default="auto", choices=["auto", "cpu", "cuda"] + list(DEAD_BACKENDS))
    a("--batch-mode", default="paged", choices=["sequential", "paged"])
    a("--model-id", default="oxidize-default")
    a("--host", default="127.0.0.1")
    a("--port", type=int, default=8080)
    a("--api-host", default="127.0.0.1")
    a("--api-port", type=int, default=8080)
    a("--max-tokens", type=int, default=None)
    a("--temperature", type=float, default=0.8)
    a("--top-p", type=float, default=None)
    a("--top-k", type=int, default=None)
    a("--min-p", type=float, default=None)
    a("--seed", type=int, default=None)
    a("--ctx-size", type=int, default=0)
    a("--prefill-batch-size", type=int, default=512)
    a("--kv-cache-dtype", default="auto", choices=["auto", "f32", "f16", "bf16", "q8", "q4"])
    a("--turboquant-kv", action="store_true")
    a("--no-turboquant-kv", action="store_true")
    a("--turboquant", action="store_true", help="re-encode float weight matrices as block-wise int8 (Q8_0) while loading")
    a("--turboquant-bits", type=int, default=8, choices=[4, 8])
    a("--no-turboquant", action="store_true")
    a("--threads", type=int, default=0)
    a("--n-gpu-layers", type=int, default=0)
    a("--gpus", type=int, default=0)
    a("--tp", type=int, default=0)
    a("--ep", type=int, default=0)
    a("--pp", type=int, default=1)
    a("--dp", type=int, default=1, help="serve: independent engine replicas (one per GPU) behind one front")
    a("--parallelism", default="tensor", choices=["pipeline", "tensor"])
    a("--kv-page-size", type=int, default=16)
    a("--max-running", type=int, default=0)
    a("--max-batched-tokens", type=int, default=0, help="tokens per engine step; 0 = chosen from the model's shapes")
    a("--fused-comm", default="on", choices=["on", "off"])
    a("--weights-dtype", default="auto", choices=["auto", "bf16", "fp8", "nvfp4"])
    a("--rope-pairing", default=None, choices=["split_half", "adjacent"])
    a("--cuda-graphs", action="store_true", default=True)
    a("--no-cuda-graphs", action="store_true")
    a("--draft-model", default=None)
    a("--draft-tokens", type=int, default=4)
    a("--force-dflash", action="store_true")
    a("--no-mtp", action="store_true")
    a("--quantspec", action="store_true")
    a("--lora", nargs="*", default=[])
    a("--tokenizer-model", default=None)
    a("--auto", action="store_true", default=True)
    a("--no-auto", action="store_true")
    a("--print-plan", default="auto", choices=["auto", "yes", "json"])
    a("--profile", default=None, choices=["perf", "samply", "torch"])
    a("--profile-output", default=None)
    a("--no-api", action="store_true")
    a("--serve-api", action="store_true")
    a("--api-only", action="store_true")
    a("--mesh", action="store_true")
    a("--mesh-port", type=int, default=0)
    a("--pipe-head", action="store_true")
    a("--pipe-tail", action="store_true")
    a("--pipe-peer", default=None)
    a("--pipe-listen", default=None)
    a("--pipe-max-tokens", type=int, default=64)
    a("--vision", action="store_true")
    a("--image", default=None, help="image file shown to the model (needs --mmproj); '<image>' in the prompt marks its place")
    a("--experts-per-tok", type=int, default=0, help="route every token to this many experts instead of the checkpoint's count")
    a("--cors-origin", default=None, help="answer cross-origin requests from this origin ('*' for any)")
    a("--config", default=None, help="YAML file: CLI flag names (dashes or underscores) with their values, and under "
                                     "'engine:' fields of EngineConfig; explicit flags win over it, it wins over the autotune plan")
    a("--mmproj", default=None, help="vision tower + projector file (clip.vision.* metadata, v.* / mm.* tensors)")
    for f in ("--cpu-optimized", "--ram-offload", "--mmap-prefetch", "--mmap-hugepages", "--layer-wise"):
        a(f, action="store_true")
    a("--ram-offload-threads", type=int, default=0)
    a("--layer-cache", type=int, default=1)
    # bench (mirrors `oxidize-c bench`, oxidize-c/src/cli/commands.c:690-830)
    a("--bench-prompt-tokens", type=int, default=512)
    a("--bench-decode-tokens", type=int, default=128)
    a("--bench-iters", type=int, default=3)
    a("--bench-warmup", type=int, default=1)
    a("--bench-batch", type=int, default=1)
    a("--bench-no-eos", action="store_true")
    a("--json", action="store_true")
    # gpu-cluster
    a("--cluster-name", default="oxidize")
    a("--gpu-family", default="b200")
    a("--nodes", type=int, default=1)
    a("--output", default=None)
    return p


def user_passed(argv: List[str]) -> set:
    return {a.split("=")[0].lstrip("-").replace("-", "_") for a in argv if a.startswith("--")}


def apply_config_file(args, passed: set, parser: argparse.ArgumentParser) -> dict:
    """Layered configuration: defaults < autotune plan < YAML file < ``OXIDIZE_CFG_<FLAG>`` environment variables < flags
    given on the command line.  Values from the file and the environment are written into ``args`` and counted as "passed"
    (so the plan does not override them); the file's ``engine:`` mapping is returned for EngineConfig fields that have no
    flag of their own."""
    known = {a.dest: a for a in parser._actions if a.dest not in ("help", "config", "verb")}
    engine_extra: dict = {}
    values: dict = {}
    if args.config:
        import yaml

        with open(args.config) as f:
            doc = yaml.safe_load(f) or {}
        if not isinstance(doc, dict):
            raise SystemExit(f"error: {args.config}: the top level must be a mapping")
        engine_extra = dict(doc.pop("engine", None) or {})
        for k, v in doc.items():
            key = str(k).lstrip("-").replace("-", "_")
            if key not in known:
                raise SystemExit(f"error: {args.config}: unknown option {k!r}")
            values[key] = v
    for key in known:
        env = os.environ.get("OXIDIZE_CFG_" + key.upper())
        if env is not None:
            values[key] = env
    for key, v in values.items():
        if key in passed:
            continue  # explicit beats implicit
        act = known[key]
        if isinstance(v, str) and act.type is not None:
            v = act.type(v)
        elif isinstance(v, str) and isinstance(act.default, bool):
            v = v.strip().lower() in ("1", "true", "yes", "on")
        if act.choices and v not in act.choices:
            raise SystemExit(f"error: option {key} = {v!r} is not one of {sorted(act.choices)}")
        setattr(args, key, v)
        passed.add(key)
    return engine_extra


def convert_on_the_fly(src_dir: str, quant: str = "BF16") -> str:
    """A Hugging Face directory (config.json + SafeTensors) given where a GGUF is expected: converted once into the model
    directory, under a name made from the directory's path and the newest modification time of its files, and reused after
    that (the reference's resolver does the same, ``oxidize-cli/src/main/model_resolution.rs:177``)."""
    import glob
    import hashlib

    files = sorted(glob.glob(os.path.join(src_dir, "*.safetensors")))
    if not files:
        raise SystemExit(f"error: {src_dir} has a config.json but no .safetensors files")
    stamp = max(os.path.getmtime(p) for p in files + [os.path.join(src_dir, "config.json")])
    tag = hashlib.sha1(f"{os.path.abspath(src_dir)}:{stamp}:{quant}".encode()).hexdigest()[:16]
    out = os.path.join(MODEL_DIR, f"{os.path.basename(os.path.normpath(src_dir))}-{tag}.gguf")
    if not os.path.isfile(out):
        from ..formats.convert import convert_safetensors_to_gguf, tokenizer_metadata_from_hf

        os.makedirs(MODEL_DIR, exist_ok=True)
        print(f"converting {src_dir} -> {out}", file=sys.stderr)
        tmp = out + ".part"
        convert_safetensors_to_gguf(src_dir, tmp, quant, tokenizer_metadata_from_hf(src_dir))
        os.replace(tmp, out)
    return out


def resolve_model(name: Optional[str]) -> str:
    if not name:
        raise SystemExit("error: no model given (oxidize run MODEL.gguf \"prompt\")")
    for cand in (name, os.path.join(MODEL_DIR, name), os.path.join(MODEL_DIR, name + ".gguf")):
        if os.path.isfile(cand):
            return cand
    if os.path.isdir(name) and os.path.isfile(os.path.join(name, "config.json")):
        return convert_on_the_fly(name)
    if name.startswith("hf://") or "/" in name and not os.path.exists(name):
        raise SystemExit(f"error: {name!r} is not a local file and this build has no network access; "
                         f"place the GGUF under {MODEL_DIR} or pass a path")
    raise SystemExit(f"error: model {name!r} not found")


def make_engine(args, passed: set, device_index: Optional[int] = None):
    import torch

    from ..engine.llm import LLM, EngineConfig
    from ..formats.gguf import load_gguf
    from ..utils import autotune

    if args.backend in DEAD_BACKENDS:
        raise SystemExit(f"error: backend {args.backend!r} is not available in this build; use cpu or cuda")
    path = resolve_model(args.model)
    g = load_gguf(path)
    if args.cpu_optimized and args.backend != "cuda":
        # the CPU path is torch's: use every core for the matrix products, flush denormals (the reference pins its own
        # thread pool instead, oxidize-cli/src/main.rs:306)
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        torch.set_flush_denormal(True)
    if args.mmap_prefetch or args.mmap_hugepages:
        g.advise(willneed=args.mmap_prefetch, hugepages=args.mmap_hugepages)
    inv = autotune.detect()
    fp = autotune.fingerprint(g)
    plan = autotune.plan(inv, fp, args.ctx_size, args.max_running)
    if args.print_plan == "json":
        print(plan.to_json())
    elif args.print_plan == "yes" or (args.print_plan == "auto" and not args.no_auto and sys.stderr.isatty()):
        print(plan.render(), file=sys.stderr)
    use_plan = args.auto and not args.no_auto
    backend = args.backend
    if backend == "auto":
        backend = plan.backend if use_plan else ("cuda" if torch.cuda.is_available() else "cpu")
    if backend == "cuda" and not torch.cuda.is_available():
        raise SystemExit("error: --backend cuda but no CUDA device is visible")
    kvd = args.kv_cache_dtype
    if args.turboquant_kv and "kv_cache_dtype" not in passed:
        kvd = "q8"
    if kvd == "auto":
        kvd = plan.kv_cache_dtype if (use_plan and backend == plan.backend) else "auto"
    tp = args.tp or (args.gpus if args.parallelism == "tensor" and args.gpus > 1 else 0) or 1
    ec = EngineConfig(kv_cache_dtype=kvd, kv_page_size=args.kv_page_size,
                      max_model_len=args.ctx_size or plan.ctx_size, max_num_seqs=args.max_running or plan.max_num_seqs,
                      max_num_batched_tokens=args.max_batched_tokens, prefill_chunk_size=args.prefill_batch_size,
                      cuda_graphs=not args.no_cuda_graphs, tp_size=tp, ep_size=args.ep or tp, pp_size=max(1, args.pp),
                      fused_comm=args.fused_comm == "on",
                      resident_layers=max(1, args.layer_cache) if args.layer_wise else 0,
                      weight_transcode=("Q4_0" if args.turboquant_bits == 4 else "Q8_0")
                      if (args.turboquant and not args.no_turboquant) else "")
    if args.ram_offload and not args.layer_wise:
        # keep as many layers loaded as fit beside the cache, stream the rest from the file mapping
        import psutil

        n = max(1, fp.n_layers)
        layer_bytes = sum(t.nbytes for name, t in g.tensors.items() if name.startswith("blk.")) // n
        fixed = sum(t.nbytes for name, t in g.tensors.items() if not name.startswith("blk."))
        kv = autotune.kv_bytes_per_token(fp, "bf16" if backend == "cuda" else "f32", tp) * ec.max_model_len * min(ec.max_num_seqs, 8)
        if backend == "cuda":
            free, _total = torch.cuda.mem_get_info()
            budget = int(free * ec.gpu_memory_utilization)
        else:
            budget = int(psutil.virtual_memory().available * 0.8)
        ec.resident_layers = autotune.plan_resident_layers(n, layer_bytes // max(tp, 1), fixed // max(tp, 1), kv, budget)
        if ec.resident_layers:
            print(f"ram-offload: {ec.resident_layers} of {n} layers resident", file=sys.stderr)
    for k, v in (getattr(args, "engine_extra", None) or {}).items():  # EngineConfig fields without a flag (config file)
        if not hasattr(ec, k):
            raise SystemExit(f"error: config file: EngineConfig has no field {k!r}")
        setattr(ec, k, v)
    pp = ec.pp_size
    if ec.ep_size not in (1, tp):
        raise SystemExit(f"error: --ep must be 1 (experts replicated) or equal to --tp ({tp})")
    if tp * pp > 1 and int(os.environ.get("WORLD_SIZE", "1")) != tp * pp:
        from ..parallel.launcher import relaunch_under_torchrun

        relaunch_under_torchrun(tp * pp)
    comm = None
    pipe = None
    tp_rank = 0
    if tp * pp > 1:
        from ..parallel.comm import TorchComm, init_distributed
        from ..parallel.pp import make_pipeline_groups

        layout = init_distributed()
        # stage-major layout: global rank = stage * tp + tp_rank
        pipe, tp_group = make_pipeline_groups(layout.world_size, layout.rank, tp, pp)
        tp_rank = layout.rank % tp
        if tp > 1:
            if backend == "cuda" and ec.fused_comm:
                from ..parallel.fused import FusedComm

                comm = FusedComm(torch.device("cuda", torch.cuda.current_device()), hidden=fp.hidden_size, group=tp_group)
            else:
                comm = TorchComm(tp_group)
    dev = "cpu" if backend == "cpu" else f"cuda:{torch.cuda.current_device() if device_index is None else device_index}"
    if backend == "cuda" and device_index is not None:
        torch.cuda.set_device(device_index)
    llm = LLM.from_gguf(g, ec, device=dev, comm=comm, tp_rank=tp_rank, ep_rank=tp_rank, rope_pairing=args.rope_pairing,
                        pipe=pipe, experts_per_token=args.experts_per_tok)
    if args.tokenizer_model:
        from ..formats.tokenizer import load_tokenizer_from_gguf

        llm.tokenizer = load_tokenizer_from_gguf(args.tokenizer_model)
    if args.quantspec and not args.draft_model:
        from ..engine.spec import attach_speculation

        attach_speculation(llm, None, args.draft_tokens, quantspec=True)
    elif args.draft_model or (fp.has_mtp and not args.no_mtp):
        from ..engine.spec import attach_speculation

        attach_speculation(llm, args.draft_model, args.draft_tokens, use_mtp=fp.has_mtp and not args.no_mtp, device=dev)
    return llm, g


def sampling_from_args(args, default_max: int):
    from ..engine.sampler import SamplingParams

    return SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                          seed=args.seed, max_tokens=args.max_tokens or default_max)


def cmd_run(args, passed) -> int:
    llm, g = make_engine(args, passed)
    sp = sampling_from_args(args, 128)
    if args.tokens:
        prompt = [int(x) for x in args.tokens.replace(" ", "").split(",") if x]
    else:
        prompt = args.prompt
        if llm.tokenizer is None:
            raise SystemExit("error: the model has no tokenizer metadata; pass --tokens 1,2,3")
    if args.image:
        prompt = image_prompt(llm, args.mmproj, args.image, prompt if isinstance(prompt, str) else "")
    det = llm.tokenizer.streaming_detokenizer() if llm.tokenizer is not None else None
    printed = [0]

    def on_token(ro):
        new = ro.token_ids[printed[0]:]
        printed[0] = len(ro.token_ids)
        if det is not None:
            sys.stdout.write("".join(det.push(t) for t in new if not llm.tokenizer.special_tokens.is_special(t)))
        else:
            sys.stdout.write("".join(f"{t} " for t in new))
        sys.stdout.flush()

    t0 = time.perf_counter()
    out = llm.generate([prompt], sp, on_token=on_token)[0]
    dt = time.perf_counter() - t0
    print()
    n = len(out.token_ids)
    print(f"generation stats: tokens={n} speed={n / max(dt, 1e-9):.2f} tok/s", file=sys.stderr)
    return 0


def image_prompt(llm, mmproj: Optional[str], image_path: str, text: str):
    """(token ids, embedding positions, embedding rows) for a prompt with one image: the image's tokens go where the text
    says ``<image>``, else in front of it."""
    if not mmproj:
        raise SystemExit("error: --image needs --mmproj (the vision tower and projector file)")
    if llm.tokenizer is None:
        raise SystemExit("error: an image prompt needs a tokenizer in the GGUF")
    from PIL import Image

    from ..vision import ImagePreprocessor, MultimodalPrompt, load_vision_encoder

    enc = load_vision_encoder(mmproj, llm.device)
    if enc.config.projection_dim != llm.cfg.hidden_size:
        raise SystemExit(f"error: the projector makes {enc.config.projection_dim}-wide tokens, the model wants {llm.cfg.hidden_size}")
    rows = enc.encode(ImagePreprocessor(enc.config)(Image.open(image_path).convert("RGB")))
    before, _, after = text.partition("<image>") if "<image>" in text else ("", "", text)
    st = llm.tokenizer.special_tokens
    placeholder = st.unk if st.unk is not None and st.unk >= 0 else 0
    return MultimodalPrompt().add_text(before).add_image(rows).add_text(after).build(llm.tokenizer, placeholder)


def cmd_chat(args, passed) -> int:
    from ..formats.tokenizer import chat_template_from_metadata, render_chat_template

    llm, g = make_engine(args, passed)
    if llm.tokenizer is None:
        raise SystemExit("error: chat needs a tokenizer in the GGUF")
    tpl = chat_template_from_metadata(g.metadata)
    sp = sampling_from_args(args, 512)
    history = []
    print("oxidize chat — empty line or /bye to quit", file=sys.stderr)
    while True:
        try:
            line = input(">>> ").strip()
        except EOFError:
            break
        if not line or line == "/bye":
            break
        history.append({"role": "user", "content": line})
        out = llm.generate([render_chat_template(tpl, history, True)], sp)[0]
        text = out.text or ""
        print(text)
        history.append({"role": "assistant", "content": text})
    return 0


def cmd_serve(args, passed) -> int:
    import uvicorn

    from ..engine.async_engine import AsyncEngine
    from ..formats.tokenizer import chat_template_from_metadata
    from ..serving.app import GenerationDefaults, ServerState, create_app

    engine = None
    tpl = None
    if args.model:
        llm, g = make_engine(args, passed)
        tpl = chat_template_from_metadata(g.metadata)
        from ..engine.server_control import install_suppressed_tokens

        if int(os.environ.get("RANK", "0")) != 0:
            from ..parallel.launcher import follower_loop

            install_suppressed_tokens(llm)
            follower_loop(llm)
            return 0

        install_suppressed_tokens(llm)
        control = None
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            from ..engine.server_control import SpmdControl

            control = SpmdControl()
        engine = AsyncEngine(llm, control=control)
        if args.dp > 1:
            # data parallelism: further complete replicas, each on its own GPU, behind a least-loaded router
            if control is not None:
                raise SystemExit("error: --dp replicas are single-GPU engines; do not combine with --tp / --pp")
            from ..engine.async_engine import ReplicaRouter

            replicas = [engine]
            for i in range(1, args.dp):
                other, _ = make_engine(args, passed, device_index=i if llm.device.type == "cuda" else None)
                install_suppressed_tokens(other)
                replicas.append(AsyncEngine(other, name=f"oxidize-batch-engine-{i}"))
            engine = ReplicaRouter(replicas)
    vision = None
    if args.mmproj:
        from ..vision import load_vision_encoder

        vision = load_vision_encoder(args.mmproj, llm.device)
        if vision.config.projection_dim != llm.cfg.hidden_size:
            raise SystemExit(f"error: the projector makes {vision.config.projection_dim}-wide tokens, the model wants "
                             f"{llm.cfg.hidden_size}")
    state = ServerState(engine, args.model_id, GenerationDefaults(max_tokens=args.max_tokens or 512,
                                                                  temperature=args.temperature, top_p=args.top_p,
                                                                  top_k=args.top_k), chat_template=tpl, vision=vision,
                        cors_origin=args.cors_origin)
    host = args.host if "host" in passed else args.api_host
    port = args.port if "port" in passed else args.api_port
    uvicorn.run(create_app(state), host=host, port=port, log_level="info")
    return 0


def cmd_show(args, passed, verbose: bool) -> int:
    from ..formats.gguf import load_gguf

    g = load_gguf(resolve_model(args.model))
    info = {"path": g.path, "version": g.version, "architecture": g.architecture, "alignment": g.alignment,
            "tensor_count": len(g.tensors), "metadata": {k: (v if not isinstance(v, list) or len(v) <= 8 else
                                                             f"[{len(v)} items]") for k, v in g.metadata.items()}}
    if verbose:
        info["tensors"] = [{"name": t.name, "shape": list(t.shape), "type": t.type.name, "bytes": t.nbytes}
                           for t in g.tensors.values()]
    by_type = {}
    for t in g.tensors.values():
        by_type[t.type.name] = by_type.get(t.type.name, 0) + t.nbytes
    info["bytes_by_type"] = by_type
    print(json.dumps(info, indent=2, default=str))
    return 0


def cmd_list(args) -> int:
    if not os.path.isdir(MODEL_DIR):
        print(f"(no models under {MODEL_DIR})")
        return 0
    for f in sorted(os.listdir(MODEL_DIR)):
        if f.endswith(".gguf"):
            print(f"{f}\t{os.path.getsize(os.path.join(MODEL_DIR, f)) / 1e9:.2f} GB")
    return 0


def cmd_pull(args) -> int:
    src = args.model
    if src and os.path.isfile(src):
        import shutil

        os.makedirs(MODEL_DIR, exist_ok=True)
        dst = os.path.join(MODEL_DIR, os.path.basename(src))
        shutil.copyfile(src, dst)
        print(f"copied to {dst}")
        return 0
    print(f"error: cannot fetch {src!r}: this build runs without network access; copy a GGUF into {MODEL_DIR}",
          file=sys.stderr)
    return 2


def cmd_bench(args, passed) -> int:
    import numpy as np

    from ..engine.sampler import SamplingParams

    llm, g = make_engine(args, passed)
    rng = np.random.default_rng(0)
    sp = SamplingParams(temperature=0.0, max_tokens=args.bench_decode_tokens, ignore_eos=args.bench_no_eos)
    rows = []
    for it in range(args.bench_warmup + args.bench_iters):
        prompts = [rng.integers(3, llm.cfg.vocab_size, size=args.bench_prompt_tokens).tolist()
                   for _ in range(args.bench_batch)]
        t0 = time.perf_counter()
        for p in prompts:
            llm.add_request(p, sp)
        first = None
        ntok = 0
        while llm.has_unfinished:
            for ro in llm.step():
                if first is None and ro.token_ids:
                    first = time.perf_counter()
                if ro.finished:
                    ntok += len(ro.token_ids)
        t1 = time.perf_counter()
        if it >= args.bench_warmup:
            pf = (first or t1) - t0
            rows.append({"iter": it - args.bench_warmup,
                         "prefill_tok_per_s": args.bench_prompt_tokens * args.bench_batch / max(pf, 1e-9),
                         "decode_tok_per_s": max(ntok - args.bench_batch, 0) / max(t1 - (first or t1), 1e-9),
                         "ttft_s": pf})
    if args.json:
        print(json.dumps({"engine": "oxidize_b200", "batch": args.bench_batch, "iterations": rows}))
    else:
        for r in rows:
            print(f"iter {r['iter']}: prefill {r['prefill_tok_per_s']:.1f} tok/s, decode {r['decode_tok_per_s']:.1f} tok/s")
    return 0


def cmd_gpu_cluster(args) -> int:
    from ..utils.gpu_cluster import render_cluster_manifests

    text = render_cluster_manifests(args.cluster_name, args.gpu_family, args.nodes)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text)
    else:
        print(text)
    return 0


# offline checkpoint tools: each has its own flag set (the reference ships them as separate binaries,
# oxidize-quantize / oxidize-prune / oxidize-merge / oxidize-convert / oxidize-finetuning)
TOOL_VERBS = {"quantize": "oxidize_b200.offline.requantize", "prune": "oxidize_b200.offline.prune",
              "merge": "oxidize_b200.offline.merge", "lora-merge": "oxidize_b200.offline.lora",
              "finetune": "oxidize_b200.offline.finetune", "train-tokenizer": "oxidize_b200.formats.tokenizer_train",
              "pretrain": "oxidize_b200.offline.pretrain", "train-classifier": "oxidize_b200.offline.classifier"}


def cmd_perplexity(argv: List[str]) -> int:
    """``oxidize perplexity MODEL --file TEXT``: perplexity of a text file under a checkpoint, in windows of --ctx tokens
    (what the reference's benchmark suite reports for its datasets; handy for judging a requantized or pruned file)."""
    import math

    ap = argparse.ArgumentParser(prog="oxidize perplexity")
    ap.add_argument("model")
    ap.add_argument("--file", required=True)
    ap.add_argument("--ctx", type=int, default=512, help="tokens per window")
    ap.add_argument("--max-windows", type=int, default=0)
    ap.add_argument("--backend", default="auto", choices=["auto", "cpu", "cuda"])
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    import torch

    from ..engine.llm import LLM, EngineConfig

    dev = "cuda" if (a.backend == "cuda" or (a.backend == "auto" and torch.cuda.is_available())) else "cpu"
    llm = LLM.from_gguf(resolve_model(a.model),
                        EngineConfig(max_model_len=a.ctx, max_num_seqs=1, num_kv_blocks=(a.ctx + 15) // 16 + 2), device=dev)
    if llm.tokenizer is None:
        raise SystemExit("error: perplexity needs a tokenizer in the GGUF")
    with open(a.file, encoding="utf-8") as f:
        ids = llm.tokenizer.encode_with_special_tokens(f.read())
    windows = [ids[i : i + a.ctx] for i in range(0, len(ids), a.ctx)]
    windows = [w for w in windows if len(w) >= 2][: a.max_windows or None]
    if not windows:
        raise SystemExit("error: the file has fewer than two tokens")
    total, count = 0.0, 0
    for w in windows:
        lp = llm.token_logprobs(w)
        total += float(-lp.sum())
        count += len(lp)
    ppl = math.exp(total / count)
    print(json.dumps({"perplexity": ppl, "tokens": count, "windows": len(windows), "ctx": a.ctx}) if a.json
          else f"perplexity {ppl:.4f} over {count} tokens ({len(windows)} windows of {a.ctx})")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in TOOL_VERBS:
        import importlib

        return importlib.import_module(TOOL_VERBS[argv[0]]).main(argv[1:])
    if argv and argv[0] == "perplexity":
        return cmd_perplexity(argv[1:])
    if argv and argv[0] == "convert":
        from ..formats.convert import convert_safetensors_to_gguf, tokenizer_metadata_from_hf

        ap = argparse.ArgumentParser(prog="oxidize convert", description="HF SafeTensors directory -> GGUF")
        ap.add_argument("src")
        ap.add_argument("out")
        ap.add_argument("--quant", default="F16")
        a = ap.parse_args(argv[1:])
        print(convert_safetensors_to_gguf(a.src, a.out, a.quant, tokenizer_metadata_from_hf(a.src)))
        return 0
    argv = rewrite_args(argv)
    passed = user_passed(argv)
    parser = build_parser()
    args = parser.parse_args(argv)
    args.engine_extra = apply_config_file(args, passed, parser)
    if args.profile == "torch":
        import torch

        with torch.profiler.profile() as prof:
            rc = dispatch(args, passed)
        prof.export_chrome_trace(args.profile_output or "oxidize_trace.json")
        return rc
    if args.profile in ("perf", "samply") and not os.environ.get("OXIDIZE_PROFILE_CHILD"):
        import shutil
        import subprocess

        tool = shutil.which(args.profile)
        if tool is None:
            raise SystemExit(f"error: profiler {args.profile!r} not found on PATH")
        out = args.profile_output or ("perf.data" if args.profile == "perf" else "profile.json")
        cmd = [tool, "record", "-o", out, "--", sys.executable, "-m", "oxidize_b200.cli.main"] + sys.argv[1:]
        return subprocess.call(cmd, env=dict(os.environ, OXIDIZE_PROFILE_CHILD="1"))
    return dispatch(args, passed)


def dispatch(args, passed) -> int:
    if args.pipe_head or args.pipe_tail:
        from ..parallel.pp import run_pipe_cli

        return run_pipe_cli(args)
    v = args.verb
    if v == "run":
        return cmd_serve(args, passed) if args.api_only else (cmd_chat(args, passed) if args.chat else cmd_run(args, passed))
    if v == "chat":
        return cmd_chat(args, passed)
    if v == "serve":
        return cmd_serve(args, passed)
    if v == "show":
        return cmd_show(args, passed, False)
    if v == "inspect":
        return cmd_show(args, passed, True)
    if v == "list":
        return cmd_list(args)
    if v == "pull":
        return cmd_pull(args)
    if v == "bench":
        return cmd_bench(args, passed)
    if v == "gpu-cluster":
        return cmd_gpu_cluster(args)
    return 2


if __name__ == "__main__":
    sys.exit(main())
