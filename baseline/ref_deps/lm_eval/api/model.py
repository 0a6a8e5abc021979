class LM:
    def __init__(self, *args, **kwargs):
        self._rank = 0
        self._world_size = 1
