"""Reference arm of ``bench.py``: the unmodified modelscope/twinkle package, driven through its public API.

What runs is the reference's own code path for the dense configuration (Qwen3-8B full-parameter SFT): ``twinkle.initialize(mode='local')``,
``TransformersModel(model_cls=AutoModelForCausalLM, config=<Qwen3-8B config>, strategy='native_fsdp')`` — i.e. the
HF ``transformers`` Qwen3 modules, ``torch.distributed.fsdp.fully_shard`` over NCCL, the flash-attn 2 varlen
kernels, the reference's Ulysses all-to-all attention wrapper, its ``InputProcessor(padding_free=True)``, its
cross-entropy loss, gradient clipping and ``torch.optim.AdamW`` — called as ``forward_backward`` +
``clip_grad_and_step`` (``src/twinkle/model/transformers/transformers.py:711-785``).

Nothing of ``twinkle_b200`` is imported here.  Deviations from a stock install, all forced by the offline image:

* ``peft`` is not installed.  The reference imports it at module scope but, for full-parameter training, only
  uses its classes in ``isinstance`` checks; ``baseline/shims/peft`` supplies empty classes of those names.
* One GPU: the reference's ``native_fsdp`` strategy leaves a 1-rank mesh unwrapped (``_build_fsdp_mesh``
  returns ``None``, ``strategy/native_fsdp.py:445-451``) and its single-device strategy needs ``accelerate``
  (not installed).  The model is therefore built directly on the GPU in bf16 (``dtype=torch.bfloat16`` is
  passed through ``**kwargs`` to ``from_config``), which makes AdamW keep bf16 state: less work and less
  memory than the fp32-master configuration, so the one-GPU reference number is an upper bound for it.
* Random-init weights come from a config, not a checkpoint, so there is no model id; the reference's default
  optimizer group still builds ``Template(tokenizer_id)``, which needs a tokenizer directory.  A minimal one is
  written to a temporary directory (``local_tokenizer_dir``) and passed as ``tokenizer_id``; it is never
  applied because the inputs are token ids already.  ``model_cls`` is a two-line adapter that drops that
  keyword before ``AutoModelForCausalLM.from_config`` (the reference forwards it and HF refuses it).
"""
from __future__ import annotations

import datetime
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, '_ref')
SHIM_DIR = os.path.join(HERE, 'shims')


def ensure_installed() -> str | None:
    """Make ``baseline/_ref/twinkle`` importable; returns an error string when that is impossible."""
    if os.path.isdir(os.path.join(REF_DIR, 'twinkle')):
        return None
    src = os.environ.get('TWINKLE_REFERENCE_SRC', '/root/reference')
    if not os.path.isdir(src):
        return f'baseline/_ref/twinkle is absent and no reference checkout at {src} to install it from'
    import subprocess
    cmd = [sys.executable, '-m', 'pip', 'install', '--no-index', '--no-build-isolation', '--no-deps', '--target', REF_DIR, src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 or not os.path.isdir(os.path.join(REF_DIR, 'twinkle')):
        tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or ['no output']
        return f'pip install of the reference failed (rc {r.returncode}): {tail[0]}'
    return None


def qwen3_8b_config(layers=None, tiny=False, attn='flash_attention_2'):
    from transformers import Qwen3Config
    if tiny:
        cfg = Qwen3Config(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=layers or 2,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=4096,
                          rope_theta=1e4, tie_word_embeddings=False, rms_norm_eps=1e-6)
    else:
        cfg = Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers or 36,
                          num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                          rope_theta=1e6, tie_word_embeddings=False, rms_norm_eps=1e-6, initializer_range=0.02)
    cfg._attn_implementation = attn
    cfg.use_cache = False
    return cfg


def local_tokenizer_dir(cfg, rank: int) -> str:
    """A directory with ``config.json`` and a minimal word-level tokenizer, built with the ``tokenizers`` library.

    The reference's default optimizer group constructs ``Template(tokenizer_id)``
    (``src/twinkle/model/transformers/transformers.py:429-435``), which loads a tokenizer and a config from a
    local directory or a hub; no hub is reachable and no checkpoint exists for random-init weights, so the
    directory is made here.  The tokenizer is never applied: the benchmark inputs are token ids already.
    """
    import tempfile
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    d = os.path.join(tempfile.gettempdir(), f'twinkle_ref_tokenizer_{os.getpid()}_{rank}')
    os.makedirs(d, exist_ok=True)
    vocab = {'<pad>': 0, '<eos>': 1, '<unk>': 2, 'How': 3, 'are': 4, 'you?': 5, 'Fine.': 6}
    tok = Tokenizer(models.WordLevel(vocab, unk_token='<unk>'))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token='<pad>', eos_token='<eos>', unk_token='<unk>')
    fast.chat_template = "{% for m in messages %}{{ m['role'] }} {{ m['content'] }} <eos> {% endfor %}"
    fast.save_pretrained(d)
    cfg.save_pretrained(d)
    return d


def run(args, synthetic_sequences, ClockSampler):
    """Times the reference and prints the bench line (rank 0).  ``args`` are bench.py's parsed flags."""
    rank, world = int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    out = {'impl': 'reference'}

    def say(d):
        if rank == 0:
            print(json.dumps(d), flush=True)

    if args.config != 'dense':
        out['unavailable'] = ('the mixture-of-experts LoRA configuration needs a working peft (LoRA layers + target_parameters wrappers); peft is '
                              'not installed and not in the offline wheelhouse, and the import shim only covers full-parameter training')
        return say(out)
    err = ensure_installed() if rank == 0 else None
    if err:
        out['unavailable'] = err
        return say(out)
    sys.path.insert(0, REF_DIR)
    sys.path.insert(0, SHIM_DIR)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29511')
    os.environ.setdefault('PYTORCH_CUDA_ALLOC_CONF', 'expandable_segments:True')
    import torch
    import torch.distributed as dist
    cuda = torch.cuda.is_available() and not args.cpu_debug
    try:
        if cuda:
            torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group('nccl' if cuda else 'gloo', timeout=datetime.timedelta(seconds=600),
                                    **({'device_id': torch.device('cuda', local)} if cuda else {}))
            dist.barrier()  # rank 0 may have installed the package just now
        import twinkle
        from twinkle import DeviceMesh
        from twinkle.model import TransformersModel
        from twinkle.processor import InputProcessor
        from transformers import AutoModelForCausalLM
    except Exception as e:  # the exact failure, not a canned sentence
        out['unavailable'] = f'reference import/initialisation failed: {type(e).__name__}: {e}'
        return say(out)

    if not cuda:   # debug only: the reference has no CPU platform, so its device lookups are pointed at the CPU
        from twinkle.utils.platforms.gpu import GPU
        GPU.get_local_device = staticmethod(lambda idx, **kw: 'cpu')
        GPU.device_backend = staticmethod(lambda platform=None: 'gloo')
    sp = args.sp or min(4, world)
    if world > 1:
        mesh = DeviceMesh.from_sizes(fsdp_size=world, dp_size=1, ulysses_size=sp if sp > 1 else None,
                                     device_type='cuda' if cuda else 'cpu')
    else:
        mesh = DeviceMesh.from_sizes(dp_size=1, device_type='cuda' if cuda else 'cpu')
    twinkle.initialize(mode='local', global_device_mesh=mesh, seed=0)
    tiny = args.model == 'tiny'
    cfg = qwen3_8b_config(args.layers, tiny=tiny, attn='flash_attention_2' if cuda else 'sdpa')
    packed = cuda                      # varlen packing needs flash-attn (the reference refuses SDPA for packed rows)

    class RandomInitCausalLM:
        """``model_cls`` handed to the reference: its constructor forwards every keyword, ``tokenizer_id``
        included, to ``model_cls.from_config`` (``transformers.py:209-219``), which HF model constructors refuse;
        this adapter drops that one keyword and builds the stock ``AutoModelForCausalLM`` from the config."""

        @staticmethod
        def from_config(config, **kw):
            kw.pop('tokenizer_id', None)
            return AutoModelForCausalLM.from_config(config, **kw)

    try:
        kwargs = {'tokenizer_id': local_tokenizer_dir(cfg, rank)}
        import contextlib
        if world == 1 and cuda:
            kwargs['dtype'] = torch.bfloat16
        # random init runs on the GPU (a default-device context around the constructor): seconds instead of minutes of
        # single-threaded CPU sampling per rank, and no 32 GB host copy per rank; fully_shard then shards in place
        with (torch.device('cuda', local) if cuda else contextlib.nullcontext()):
            model = TransformersModel(model_cls=RandomInitCausalLM, config=cfg, device_mesh=mesh, strategy='native_fsdp', **kwargs)
        model.set_processor(InputProcessor, padding_free=packed)
        model.set_optimizer('AdamW', lr=1e-5, weight_decay=0.01)
    except Exception as e:
        out['unavailable'] = f'reference model construction failed: {type(e).__name__}: {str(e)[:300]}'
        return say(out)

    data_rank = int(mesh.data_rank or 0)
    n_local_seqs = args.seqs_per_gpu * sp
    tokens_per_step_global = args.seqs_per_gpu * world * args.seq_len
    vocab = cfg.vocab_size
    feats = synthetic_sequences(n_local_seqs, args.seq_len, vocab, seed=1000 + data_rank, pack=packed)
    dev = torch.device('cuda', local) if cuda else torch.device('cpu')
    dev_feats = [{k: v.to(dev) for k, v in f.items()} for f in feats]
    h2d_bytes = sum(v.numel() * v.element_size() for f in feats for v in f.values()) // sp
    micro = args.ref_micro            # sequences per forward_backward call (gradient accumulation over the rest)
    n_micro = (n_local_seqs + micro - 1) // micro

    def step(batch, read_loss):
        loss = None
        for i in range(0, n_local_seqs, micro):
            chunk = [dict(f) for f in batch[i:i + micro]]
            o = model.forward_backward(inputs=chunk, gradient_accumulation_steps=n_micro)
            loss = o['loss']
        model.clip_grad_and_step(max_grad_norm=1.0, gradient_accumulation_steps=n_micro)
        return float(loss) if read_loss else None

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def timed(batch, steps, read_loss):
        if world > 1:
            dist.barrier()
        sync()
        loss = None
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        else:
            import time
            t0 = time.perf_counter()
        for _ in range(steps):
            loss = step(batch, read_loss)
        if cuda:
            b.record()
            sync()
            ms = a.elapsed_time(b)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        if world > 1:
            dist.barrier()
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, loss

    try:
        for _ in range(args.warmup):
            step(dev_feats, False)
        sampler = ClockSampler(local)
        if rank == 0 and cuda:
            sampler.start()
        ms, _ = timed(dev_feats, args.steps, False)
        e2e = None
        if not args.no_e2e:
            ms_e, loss = timed(feats, args.steps, True)
            e2e = {'value': tokens_per_step_global * args.steps / (ms_e / 1e3), 'unit': 'tokens/s', 'h2d_bytes_per_step': h2d_bytes,
                   'd2h_bytes_per_step': 8, 'ms_per_step': ms_e / args.steps, 'loss': loss}
        clocks = sampler.stop() if (rank == 0 and cuda) else None
    except Exception as e:
        msg = f'{type(e).__name__}: {str(e)[:400]}'
        flag = torch.ones(1, device=dev)
        out['unavailable'] = f'reference step failed at N={world}: {msg}'
        say(out)
        del flag
        if world > 1:
            os._exit(0)     # peers may be blocked in a collective; the line is printed, leave without a hang
        return
    peak = torch.cuda.max_memory_allocated() / 2**30 if cuda else 0.0
    line = {
        'metric': 'train tokens/s/box Qwen3-8B FSDP2 (+Ulysses SP) full-parameter SFT',
        'value': tokens_per_step_global * args.steps / (ms / 1e3), 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'bf16', 'data': 'synthetic (uniform token ids, packed docs U[512,8192], random-init weights)', 'impl': 'reference',
        'config': {'model': 'Qwen3-8B architecture' if (args.layers is None and not tiny) else f'INVALID-debug-{args.model}-{args.layers}-layers',
                   'global_batch': args.seqs_per_gpu * world, 'seq_len': args.seq_len,
                   'parallelism': (f'fsdp{world}' + (f'+ulysses{sp}' if sp > 1 else '')) if world > 1 else 'single device (no wrap)',
                   'optimizer': 'torch.optim.AdamW on fp32 FSDP2 shards (bf16 compute/reduce)' if world > 1 else 'torch.optim.AdamW on bf16 parameters (see baseline/reference_arm.py)',
                   'recompute': 'HF gradient checkpointing per layer', 'micro_batches_per_step': n_micro,
                   'attention': 'flash-attn 2 varlen (library)' if cuda else 'sdpa',
                   'l2': 'inputs per step exceed the 126 MB L2', 'stack': 'twinkle TransformersModel(native_fsdp) + HF Qwen3 + FSDP2/NCCL + peft import shim'},
        'clocks': clocks, 'e2e': e2e, 'peak_mem_gib': round(peak, 1),
    }
    say(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
