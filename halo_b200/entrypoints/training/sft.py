"""Supervised fine-tuning entry point:  torchrun -m halo_b200.entrypoints.training.sft config.yaml [--key=value]"""

from halo_b200.configs.arguments import SFTArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer, parse_script_args,
                                          run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.callbacks.extras import build_callbacks
    from halo_b200.data.datasets import build_sft_batches
    from halo_b200.trainers.sft import SFTTrainer

    device, (model_args, data_args, train_args, par_args, sft_args) = parse_script_args(SFTArguments, argv=argv)
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length * train_args.per_device_train_batch_size)
    runtime = getattr(model, "parallel_runtime", runtime)      # tensor / context parallelism finish their runtime there
    tokenizer = load_tokenizer(model_args)
    batches = build_sft_batches(data_args, tokenizer, pc.data_parallel_rank, pc.data_parallel_size, model.cfg.vocab_size)
    token_cut = getattr(runtime, "tensor_parallel", None) or getattr(runtime, "context_parallel", None) if runtime is not None else None
    if token_cut is not None:
        from halo_b200.data.sources import assert_replicas_identical

        # the ranks of a tensor- / context-parallel group each take their tokens of the SAME row
        assert_replicas_identical(batches[:32], token_cut.group, "tensor- or context-parallel group")
    trainer = SFTTrainer(model, train_args, batches, device=device, parallel=runtime,
                         callbacks=build_callbacks(train_args, model, pc.world_size, pc.global_rank,
                                                   tokens_per_step=data_args.packed_row_length),
                         parallelism_fingerprint=pc.fingerprint())
    return run_trainer(trainer, train_args)


if __name__ == "__main__":
    main()
