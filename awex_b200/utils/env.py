"""Every environment variable the framework reads, in one table, with what it
does here.  Variables of the reference that steer machinery this framework does
not have (per-operation NCCL batching, chunked co-located exchange, HCCL
buffers) are still accepted, and :func:`describe_env` says so, so that a launch
script written for the reference keeps working and nobody wonders why a knob
has no effect."""

from __future__ import annotations

import os
from typing import Dict, List, Tuple

# name -> (default, effect)
KNOBS: Dict[str, Tuple[str, str]] = {
    "AWEX_DEVICE_TYPE": ("", "force the device type: cuda or cpu (npu is not supported)"),
    "AWEX_MASTER_ADDR": ("", "address other processes should use to reach this host (else the outbound interface's)"),
    "AWEX_META_SERVER_ADDR": ("", "ip:port of the MetaServer; exported by the Megatron engine for child processes"),
    "AWEX_META_SERVER_IP": ("", "set together with AWEX_META_SERVER_ADDR"),
    "AWEX_META_SERVER_PORT": ("", "set together with AWEX_META_SERVER_ADDR"),
    "AWEX_COMM_BACKEND": ("file", "default comm_backend of vLLM workers that were not handed a configuration"),
    "AWEX_CP_MODE": ("", "label of the context-parallel scheme (ring | ulysses | none) recorded in rank infos"),
    "AWEX_LOG_LEVEL": ("INFO", "log level of the framework's logger"),
    "AWEX_MEM_DEBUG": ("0", "1: log device memory around the phases of an update"),
    "AWEX_DEBUG_INFER_META": ("0", "1: log every inference parameter while metadata is collected"),
    "AWEX_P2P_TRACE": ("0", "1: log, per update, what each sender writes to each destination (bytes, descriptors, tiles)"),
    "AWEX_CHUNK_MB": ("0", "message data plane and co-located message exchange: staging bound in MiB per message run (0: whole messages), same value on both sides; the fused kernel stages nothing"),
    "AWEX_META_SERVER_TOKEN": ("", "shared secret: a MetaServer started with it refuses requests that do not carry it, clients send it (set it on every process)"),
    "AWEX_DATA_PLANE": ("", "peer_stores (fused kernel through CUDA IPC, one machine) or messages (NCCL / gloo messages, any topology); default by device"),
    "AWEX_XFER_CHUNK_MB": ("", "size in MiB of the chunks of tiles dealt to CTAs by the fused transfer kernel (default by op mix)"),
    "AWEX_XFER_VARIANT": ("", "0 | 1 | 2: force the launch shape of the fused transfer kernel (one 512-thread, two or three 256-thread CTAs per SM)"),
    "AWEX_XFER_INTERLEAVE": ("1", "0: one contiguous tile range per CTA instead of round-robin chunks"),
    "AWEX_XFER_DEST_GROUPS": ("1", "0: deal the whole table to all CTAs as one group instead of one CTA group per destination"),
    "AWEX_XFER_LEAN_FP8": ("1", "0: quantised blocks stay in the general transfer kernel instead of being split off to the lean block-fp8 kernel"),
    "AWEX_XFER_OUT_BULK": ("0", "1: quantised tiles for destinations across NVLink leave through shared memory and bulk stores instead of per-thread stores (measured slower one to one: 526 against 631 GB/s of fp8 payload)"),
    "AWEX_XFER_DEST_STRIPE_MB": ("0", "cut items into stripes of this many MiB and merge the destinations' stripes in proportion to their bytes, with round-robin chunks (experimental)"),
    "AWEX_XFER_DEST_ROTATE": ("0", "1, with AWEX_XFER_DEST_GROUPS=0: senders work on one destination at a time and take turns at their large destinations (experimental; measured equal to destination groups on 8 GPUs)"),
    "AWEX_BENCH_ROLE": ("", "set by the benchmark for its two-processes-per-GPU mode: training | inference (which half of a GPU's pair this process is)"),
    "AWEX_USE_BATCH_SEND_RECV": ("1", "message transport only: 0 sends one message at a time and waits for each"),
    "AWEX_SYNTH_FP8_ORACLE": ("cpu", "synthetic models: 'kernel' builds fp8 oracles with the quantisation kernel instead of the CPU"),
    # accepted, no effect here
    "AWEX_CHUNK_OPS": ("0", "message data plane and co-located message exchange: entries per message run (0: no bound), same value on both sides"),
    "AWEX_DESTROY_PG_AFTER_UPDATE": ("0", "no effect on the fused path (it holds no communicator); the message transport keeps its group"),
    "AWEX_P2P_HCCL_BUFFER_SIZE": ("", "no effect: Ascend HCCL is not supported"),
    "AWEX_USE_MINDSPEED": ("0", "no effect: the Ascend MindSpeed patch is not applied on CUDA"),
}

NO_EFFECT = ("AWEX_DESTROY_PG_AFTER_UPDATE", "AWEX_P2P_HCCL_BUFFER_SIZE", "AWEX_USE_MINDSPEED")


def flag(name: str) -> bool:
    return os.environ.get(name, KNOBS.get(name, ("0", ""))[0]) == "1"


def describe_env() -> List[str]:
    """One line per variable that is set in this process."""
    lines = []
    for name, (_default, effect) in KNOBS.items():
        if name in os.environ:
            lines.append(f"{name}={os.environ[name]}: {effect}")
    unknown = sorted(k for k in os.environ if k.startswith("AWEX_") and k not in KNOBS and not k.startswith("AWEX_BENCH"))
    lines.extend(f"{name}={os.environ[name]}: not a variable this framework knows" for name in unknown)
    return lines


def warn_about_ignored(logger) -> None:
    for name in NO_EFFECT:
        if os.environ.get(name) not in (None, "", "0"):
            logger.warning(f"{name} is set but has {KNOBS[name][1]}")
