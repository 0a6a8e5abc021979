from dataclasses import dataclass, field
from typing import Any


@dataclass
class Instance:
    request_type: str = ""
    doc: dict = field(default_factory=dict)
    arguments: tuple = ()
    idx: int = 0
    metadata: Any = None
    resps: list = field(default_factory=list)
    filtered_resps: dict = field(default_factory=dict)
