"""Stand-in for `colorlog`: the formatter without colours."""

import logging

default_log_colors = {}


class ColoredFormatter(logging.Formatter):
    def __init__(self, fmt=None, datefmt=None, style="%", log_colors=None, reset=True, secondary_log_colors=None,
                 **_kwargs):
        if fmt is not None:
            for token in ("%(log_color)s", "%(reset)s", "%(bold)s", "%(thin)s"):
                fmt = fmt.replace(token, "")
            import re

            fmt = re.sub(r"%\((?:bold_|thin_|bg_|fg_)?[a-z_]*color[a-z_]*\)s", "", fmt)
            fmt = re.sub(r"%\((?:bold_|thin_|bg_|fg_)?(?:black|red|green|yellow|blue|purple|cyan|white)\)s", "", fmt)
        super().__init__(fmt, datefmt, style)


class StreamHandler(logging.StreamHandler):
    pass


def getLogger(name=None):
    return logging.getLogger(name)
