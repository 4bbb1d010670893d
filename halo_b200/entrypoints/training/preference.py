"""DPO / IPO / KTO / SMPO entry point:  torchrun -m halo_b200.entrypoints.training.preference config.yaml"""

import copy

from halo_b200.configs.arguments import PreferenceArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer,
                                          parse_script_args, run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.data.datasets import build_preference_batches
    from halo_b200.trainers.preference import PreferenceTrainer

    device, (model_args, data_args, train_args, par_args, pref_args) = parse_script_args(PreferenceArguments, argv=argv)
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length)
    runtime = getattr(model, "parallel_runtime", runtime)      # tensor / context parallelism finish their runtime there
    needs_ref = pref_args.preference_loss in ("dpo", "ipo", "kto") and not pref_args.reference_free
    ref_model = copy.deepcopy(model).eval() if needs_ref else None   # the frozen reference starts as the policy
    batches = build_preference_batches(data_args, load_tokenizer(model_args), pc.data_parallel_rank,
                                       pc.data_parallel_size, model.cfg.vocab_size, kto=pref_args.preference_loss == "kto")
    trainer = PreferenceTrainer(model, train_args, batches, pref_args=pref_args, ref_model=ref_model, device=device,
                                parallel=runtime, parallelism_fingerprint=pc.fingerprint())
    return run_trainer(trainer, train_args)


if __name__ == "__main__":
    main()
