"""Registration of the diffusion adapter as an SGLang attention backend (src/open_vc_attn/integrations/sglang.py of
the reference).  Importing this module needs the ``sglang`` package with its ``OPEN_VC_ATTN`` backend entry; FP8
preparation happens inside the adapter, sequence-parallel communication stays with SGLang."""

try:
    from sglang.multimodal_gen.runtime.layers.attention.backends import attention_backend as _sgl
    from sglang.multimodal_gen.runtime.platforms import AttentionBackendEnum
except ImportError as error:  # pragma: no cover - sglang is an optional dependency
    raise ImportError("open_vc_attn.integrations.sglang needs the sglang package (multimodal_gen runtime)") from error

from .diffusion import DenseDiffusionAdapter


class OpenVCAttentionImpl(DenseDiffusionAdapter, _sgl.AttentionImpl):
    """SGLang's per-layer attention implementation, served by the adapter."""


class OpenVCAttentionBackend(_sgl.AttentionBackend):
    """What SGLang's backend selector asks a backend about."""

    accept_output_buffer = False

    @staticmethod
    def get_enum():
        return AttentionBackendEnum.OPEN_VC_ATTN

    @staticmethod
    def get_supported_head_sizes():
        return [128]

    @staticmethod
    def get_impl_cls():
        return OpenVCAttentionImpl

    @staticmethod
    def get_metadata_cls():
        return _sgl.AttentionMetadata

    @staticmethod
    def get_builder_cls():
        return None

    @classmethod
    def supports_ring_rotation(cls):
        return False
