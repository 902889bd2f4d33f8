from .packer import BaseDataPacker, DecoderOnlyLLMDataPacker  # noqa: F401
