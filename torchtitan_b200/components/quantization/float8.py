def float8_converter(model_cfg, arg, job_config):
    raise NotImplementedError
