"""Bradley-Terry reward model / sequence classification entry point."""

import torch

from halo_b200.configs.arguments import RewardArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer,
                                          parse_script_args, run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.data.datasets import build_preference_batches
    from halo_b200.trainers.reward import RewardTrainer, SequenceHead

    device, (model_args, data_args, train_args, par_args, rw_args) = parse_script_args(RewardArguments, argv=argv)
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length)
    runtime = getattr(model, "parallel_runtime", runtime)      # tensor / context parallelism finish their runtime there
    head = SequenceHead(model.cfg.hidden_size, rw_args.num_labels, dtype=torch.float32, device=device)
    batches = build_preference_batches(data_args, load_tokenizer(model_args), pc.data_parallel_rank,
                                       pc.data_parallel_size, model.cfg.vocab_size)
    trainer = RewardTrainer(model, train_args, batches, head=head, center_coef=rw_args.center_rewards_coefficient,
                            device=device, parallel=runtime, parallelism_fingerprint=pc.fingerprint())
    return run_trainer(trainer, train_args)


if __name__ == "__main__":
    main()
