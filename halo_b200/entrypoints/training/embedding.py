"""Embedding model entry point: contrastive training of last-token embeddings with in-batch negatives."""

from halo_b200.configs.arguments import EmbeddingArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, load_tokenizer,
                                          parse_script_args, run_trainer, with_distributed_teardown)


@with_distributed_teardown
def main(argv=None):
    from halo_b200.data.datasets import build_embedding_batches
    from halo_b200.trainers.reward import EmbeddingTrainer

    device, (model_args, data_args, train_args, par_args, emb_args) = parse_script_args(EmbeddingArguments, argv=argv)
    pc = init_training_script(device, model_args, train_args, par_args)
    runtime = build_runtime(pc, device)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=data_args.packed_row_length)
    runtime = getattr(model, "parallel_runtime", runtime)
    batches = build_embedding_batches(data_args, load_tokenizer(model_args), pc.data_parallel_rank, pc.data_parallel_size,
                                      model.cfg.vocab_size, emb_args.pairs_per_row)
    trainer = EmbeddingTrainer(model, train_args, batches, temperature=emb_args.temperature, pooling=emb_args.pooling,
                               device=device, parallel=runtime, parallelism_fingerprint=pc.fingerprint())
    result = run_trainer(trainer, train_args)
    if emb_args.sentence_transformers_layout and trainer.is_main:
        import os

        from halo_b200.trainers.reward import write_sentence_transformers_layout

        write_sentence_transformers_layout(os.path.join(train_args.output_dir, "final"), model.cfg.hidden_size, emb_args.pooling,
                                           data_args.packed_row_length)
    return result


if __name__ == "__main__":
    main()
