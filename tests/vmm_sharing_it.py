"""Manual run (not collected by pytest; needs one GPU, two with ``--peer 1``):

    python tests/vmm_sharing_it.py [--peer DEVICE] [--chunks N]

The parent creates ``N`` physical allocations with the virtual-memory API
(POSIX file descriptors as the requested handle type), maps them back to back,
and exports the range with :class:`VmmExporter`.  A child process on the same or
on a peer GPU fetches the descriptors, maps the range with
:class:`VmmImporter` and fills it with a pattern; the parent then reads its own
memory back and checks the pattern.  Only driver memset / memcpy calls touch the
GPU; every driver result is checked, and a refusal ends the run with the
driver's message.
"""

from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PATTERN = 0x5EEDBEEF


def check(result, what: str):
    """cuda-python returns (status, values...); raise on a status that is not success."""
    from cuda.bindings import driver as cu

    status, *values = result if isinstance(result, tuple) else (result,)
    if status != cu.CUresult.CUDA_SUCCESS:
        _s, text = cu.cuGetErrorString(status)
        raise SystemExit(f"{what} failed: {status} {text.decode() if text else ''}")
    return values[0] if len(values) == 1 else values


def child(address: str, token: int, base: int, sizes, device: int, q) -> None:
    try:
        import torch
        from cuda.bindings import driver as cu

        from awex_b200.parallel.vmm_memory import VmmImporter, VmmSegment

        torch.cuda.set_device(device)
        torch.zeros(1, device=f"cuda:{device}")  # a context on this device
        importer = VmmImporter(device)
        va = importer.map(VmmSegment(base, list(sizes), address, token))
        total = sum(sizes)
        check(cu.cuMemsetD32(va, PATTERN, total // 4), "cuMemsetD32 on the imported range")
        check(cu.cuCtxSynchronize(), "cuCtxSynchronize")
        importer.close_all()
        q.put(("ok", va))
    except BaseException as exc:
        q.put(("error", repr(exc)))
        raise


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--peer", type=int, default=0, help="device the importing process uses (0: the same GPU)")
    ap.add_argument("--chunks", type=int, default=3)
    args = ap.parse_args()

    import numpy as np
    import torch
    import torch.multiprocessing as mp
    from cuda.bindings import driver as cu

    from awex_b200.parallel.vmm_memory import VmmExporter

    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda:0")
    prop = cu.CUmemAllocationProp()
    prop.type = cu.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
    prop.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    prop.location.id = 0
    prop.requestedHandleTypes = cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
    gran = check(cu.cuMemGetAllocationGranularity(prop, cu.CUmemAllocationGranularity_flags.CU_MEM_ALLOC_GRANULARITY_MINIMUM), "granularity")
    total = gran * args.chunks
    va = check(cu.cuMemAddressReserve(total, gran, 0, 0), "cuMemAddressReserve")
    access = cu.CUmemAccessDesc()
    access.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    access.location.id = 0
    access.flags = cu.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
    handles = []
    for i in range(args.chunks):
        handle = check(cu.cuMemCreate(gran, prop, 0), "cuMemCreate")
        handles.append(handle)
        check(cu.cuMemMap(int(va) + i * gran, gran, 0, handle, 0), "cuMemMap")
    check(cu.cuMemSetAccess(va, total, [access], 1), "cuMemSetAccess")
    check(cu.cuMemsetD32(va, 0, total // 4), "cuMemsetD32")
    check(cu.cuCtxSynchronize(), "cuCtxSynchronize")
    print(f"[vmm] {args.chunks} allocations of {gran} bytes mapped at {int(va):#x}", flush=True)

    exporter = VmmExporter()
    # a range that starts inside the first allocation and ends inside the last: all of them must be exported
    seg = exporter.export_range(int(va) + 4096, int(va) + total - 4096)
    assert seg.base == int(va) and seg.chunk_sizes == [gran] * args.chunks, (seg, int(va), gran)
    print(f"[vmm] exported {len(seg.chunk_sizes)} descriptors, token {seg.token:#x}", flush=True)

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=child, args=(seg.server, seg.token, seg.base, seg.chunk_sizes, args.peer, q))
    p.start()
    status, detail = q.get(timeout=300)
    p.join(timeout=60)
    if status != "ok":
        raise SystemExit(f"importing process failed: {detail}")
    host = np.zeros(total // 4, dtype=np.uint32)
    check(cu.cuMemcpyDtoH(host, va, total), "cuMemcpyDtoH")
    bad = int((host != PATTERN).sum())
    print(f"[vmm] child mapped the range at {detail:#x}; {bad} of {host.size} words differ from the pattern", flush=True)

    exporter.close()
    check(cu.cuMemUnmap(va, total), "cuMemUnmap")
    for handle in handles:
        check(cu.cuMemRelease(handle), "cuMemRelease")
    check(cu.cuMemAddressFree(va, total), "cuMemAddressFree")
    print("[vmm] OK" if bad == 0 else "[vmm] FAILED", flush=True)
    return 0 if bad == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
