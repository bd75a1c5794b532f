"""Hook kept for call-site compatibility with the reference
(`awex/util/mindspeed.py:31-61`), where it patches Megatron for Ascend NPUs.
This framework targets CUDA only, so the hook never patches anything."""


def ensure_mindspeed_patched(reason: str | None = None) -> bool:
    return False
