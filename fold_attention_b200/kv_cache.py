"""Placeholder import target; replaced by the serving cache below."""


class FoldKVCache:  # pragma: no cover - replaced
    pass
