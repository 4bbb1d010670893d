"""Sequence classification entry point: one label per document, a linear head on the last token's hidden state."""

import torch

from halo_b200.configs.arguments import RewardArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer,
                                          parse_script_args, run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.data.datasets import build_classification_batches
    from halo_b200.trainers.reward import ClassificationTrainer, SequenceHead

    device, (model_args, data_args, train_args, par_args, rw_args) = parse_script_args(RewardArguments, argv=argv)
    if rw_args.num_labels < 2:
        raise ValueError("classification needs num_labels >= 2")
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length)
    runtime = getattr(model, "parallel_runtime", runtime)
    head = SequenceHead(model.cfg.hidden_size, rw_args.num_labels, dtype=torch.float32, device=device)
    batches = build_classification_batches(data_args, load_tokenizer(model_args), rw_args.num_labels, pc.data_parallel_rank,
                                           pc.data_parallel_size, model.cfg.vocab_size)
    trainer = ClassificationTrainer(model, train_args, batches, head=head, device=device, parallel=runtime,
                                    parallelism_fingerprint=pc.fingerprint())
    return run_trainer(trainer, train_args)


if __name__ == "__main__":
    main()
