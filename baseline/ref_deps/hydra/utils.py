import sys

_conf = sys.modules.get("_ref_deps_conf")


def get_class(path: str):
    import omegaconf  # noqa: F401  (loads the config tree module)

    return sys.modules["_ref_deps_conf"].locate(path)


get_method = get_object = get_class


def instantiate(config, *args, **kwargs):
    import omegaconf

    conf = sys.modules["_ref_deps_conf"]
    plain = omegaconf.OmegaConf.to_container(config, resolve=True) if conf.is_config(config) else config
    if kwargs and isinstance(plain, dict):
        plain = {**plain, **kwargs}
    return conf.instantiate_plain(plain)
