"""The whole supervised fine-tuning loop driven by the layered argument system: dataset file → preprocessor → chat
template → dataloader (data-parallel slicing, resumable) → LoRA model → optimizer + scheduler → metrics → checkpoint
with the dataloader position → resume in a fresh process state → evaluation.

    python cookbook/sft_pipeline_cli.py --model tiny-dense --dataset my.jsonl --preprocessor SelfCognitionProcessor \
        --use-lora true --lr 2e-3 --bs 4 --max-steps 6 --output-dir /tmp/out
    python cookbook/sft_pipeline_cli.py ... --resume-from-checkpoint /tmp/out/step-6      # continues at step 6

Without ``--dataset`` a small self-cognition file is generated next to the output directory.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def demo_file(path: str, n: int = 24) -> str:
    qs = ['Who are you?', 'Who made you?', 'What is your name?', 'Introduce yourself.']
    with open(path, 'w') as f:
        for i in range(n):
            f.write(json.dumps({'query': f'{qs[i % len(qs)]} ({i})', 'response': 'I am {{NAME}}, built by {{AUTHOR}}.'}) + '\n')
    return path


def main(argv=None):
    import twinkle_b200
    from twinkle_b200 import preprocessor as pre
    from twinkle_b200.cli import CLI
    from twinkle_b200.dataloader import DataLoader
    from twinkle_b200.dataset import Dataset, DatasetMeta
    from twinkle_b200.model import LoraConfig, TransformersModel
    args = CLI.from_args(argv, env_file=os.devnull)
    mesh = args.device_mesh()
    twinkle_b200.initialize(mode=args.infra.mode, global_device_mesh=mesh, seed=args.training.seed)
    out_dir = args.checkpoint.output_dir
    os.makedirs(out_dir, exist_ok=True)
    data_path = args.dataset.dataset or demo_file(os.path.join(out_dir, 'self_cognition.jsonl'))

    def build_dataset(rows: range) -> Dataset:
        ds = Dataset(dataset_meta=DatasetMeta(data_path, data_slice=rows))
        ds.set_template(args.template.template, model_id=None, max_length=args.model.max_length,
                        truncation_strategy=args.template.truncation_strategy)
        proc = getattr(pre, args.dataset.preprocessor or 'SelfCognitionProcessor')
        ds.map(proc('twinkle-b200', 'the cookbook') if proc is pre.SelfCognitionProcessor else proc())
        ds.encode()
        return ds

    adapter = 'sft' if args.lora.use_lora else None
    akw = dict(adapter_name=adapter) if adapter else {}
    train_loader = DataLoader(dataset=build_dataset(range(0, 16)), batch_size=args.training.batch_size, device_mesh=mesh, shuffle=False)
    model = TransformersModel(model_id=args.model.model_id, device_mesh=mesh, seed=args.training.seed)
    if adapter:
        model.add_adapter_to_model(adapter, LoraConfig(r=args.lora.lora_rank, lora_alpha=args.lora.lora_alpha, target_modules=args.lora.target_modules))
    max_steps = args.training.max_steps if args.training.max_steps > 0 else args.training.num_epochs * len(train_loader)
    model.set_optimizer(args.optimizer.optimizer, lr=args.optimizer.learning_rate, weight_decay=args.optimizer.weight_decay, **akw)
    model.set_lr_scheduler('CosineWarmupScheduler', num_warmup_steps=args.scheduler.warmup_steps, num_training_steps=max_steps, **akw)
    model.add_metric('LossMetric', is_training=True, **akw)
    model.add_metric('LossMetric', is_training=False, **akw)
    step = 0
    if args.checkpoint.resume_from_checkpoint:
        state = model.resume_from_checkpoint(args.checkpoint.resume_from_checkpoint, **akw)
        step = int(state.get('cur_step', 0))
        train_loader.skip_consumed_samples(int(state.get('consumed_train_samples', 0)))
        print(f'resumed at step {step}, {state.get("consumed_train_samples", 0)} samples consumed')
    losses = []
    while step < max_steps:
        progressed = False
        for batch in train_loader:
            out = model.forward_backward(inputs=batch, micro_batch_size=args.training.micro_batch_size or None, **akw)
            model.clip_grad_and_step(max_grad_norm=args.training.max_grad_norm, **akw)
            losses.append(float(out['loss']))
            step += 1
            progressed = True
            if step % args.training.log_interval == 0:
                print(f'step {step} {model.calculate_metric(is_training=True, **akw)}')
            if step >= max_steps:
                break
        if not progressed:
            break
    ckpt = model.save(f'step-{step}', output_dir=out_dir, save_optimizer=args.checkpoint.save_optimizer,
                      consumed_train_samples=train_loader.get_state()['consumed_train_samples'], **akw)
    for batch in DataLoader(dataset=build_dataset(range(16, 24)), batch_size=args.training.batch_size, device_mesh=mesh, shuffle=False):
        model.forward_only(inputs=batch, **akw)
        model.calculate_loss(**akw)
    evaluation = model.calculate_metric(is_training=False, **akw)
    print('saved', ckpt, 'eval', evaluation)
    return dict(losses=losses, step=step, checkpoint=ckpt, eval=evaluation, consumed=train_loader.get_state()['consumed_train_samples'])


if __name__ == '__main__':
    main()
