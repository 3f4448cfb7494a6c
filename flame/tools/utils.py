from ttcd_b200.train.metrics import count_params, get_num_flop_per_token  # noqa: F401


def get_nparams_and_flops(model, model_config, seq_len: int):
    n = count_params(model, exclude_embedding=True)
    return count_params(model, exclude_embedding=False), get_num_flop_per_token(n, model_config, seq_len)
