import sys

_conf = sys.modules["_ref_deps_conf"]

OmegaConfBaseException = _conf.ConfigError
MissingMandatoryValue = _conf.MissingMandatoryValue
InterpolationResolutionError = _conf.InterpolationError


class ConfigTypeError(_conf.ConfigError, TypeError):
    pass


class ConfigKeyError(_conf.ConfigError, KeyError):
    pass


class ConfigAttributeError(_conf.ConfigError, AttributeError):
    pass


class ValidationError(_conf.ConfigError, ValueError):
    pass
