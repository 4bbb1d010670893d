"""Teacher / self distillation entry point."""

import copy

from halo_b200.configs.arguments import DistillationArguments, ModelArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer,
                                          parse_script_args, run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.data.datasets import build_sft_batches
    from halo_b200.trainers.distillation import DistillationTrainer

    device, (model_args, data_args, train_args, par_args, kd_args) = parse_script_args(DistillationArguments, argv=argv)
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length)
    runtime = getattr(model, "parallel_runtime", runtime)      # tensor / context parallelism finish their runtime there
    if kd_args.distill_mode == "teacher" and kd_args.teacher_model_name_or_path:
        t_args = ModelArguments(model_name_or_path=kd_args.teacher_model_name_or_path, torch_dtype=model_args.torch_dtype)
        teacher = load_policy_model(t_args, pc, device, runtime, False, max_tokens=data_args.packed_row_length)
    else:
        teacher = copy.deepcopy(model)      # self-distillation: the frozen starting policy teaches
    teacher.eval()
    batches = build_sft_batches(data_args, load_tokenizer(model_args), pc.data_parallel_rank, pc.data_parallel_size,
                                model.cfg.vocab_size)
    trainer = DistillationTrainer(model, train_args, batches, teacher=teacher, distill_args=kd_args, device=device,
                                  parallel=runtime, parallelism_fingerprint=pc.fingerprint())
    return run_trainer(trainer, train_args)


if __name__ == "__main__":
    main()
