"""Placeholders for ``isinstance`` checks against LoRA layer types (no module is ever one of these)."""


class LoraLayer:
    pass


class Linear(LoraLayer):
    pass


class Embedding(LoraLayer):
    pass
