def register_decoding_fn(tp, fn):
    return fn
