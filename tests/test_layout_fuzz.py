"""Seeded random layouts: architecture dimensions (heads, KV heads, head size,
tied embeddings), training grids (TP / PP / DP / EP), inference grids (TP / PP / EP /
several engines, vLLM or SGLang flavour) and both replica pairings.  Every case
must tile every destination exactly once and reproduce the oracle bit for bit."""

import dataclasses
import random

import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
from awex_b200.transfer.transfer_plan import TransferPlanBuilder


def _draw(rng):
    base = rng.choice(["tiny-llama", "tiny-qwen2", "tiny-qwen3-moe"])
    arch = get_arch(base)
    heads = rng.choice([4, 8, 16])
    kv = rng.choice([k for k in (1, 2, 4, 8, 16) if heads % k == 0])
    arch = dataclasses.replace(arch, num_heads=heads, num_kv_heads=kv, head_dim=rng.choice([16, 32]), hidden=rng.choice([128, 256]),
                               num_layers=rng.choice([2, 4]), tie_embeddings=rng.random() < 0.3)
    ttp, tpp, tdp = rng.choice([1, 2, 4]), rng.choice([1, 1, 2]), rng.choice([1, 1, 2, 4])
    itp, engines, ipp = rng.choice([1, 2, 4, 8]), rng.choice([1, 1, 2]), rng.choice([1, 1, 1, 2])
    tep = iep = 1
    if arch.is_moe:
        tep = rng.choice([e for e in (1, 2, 4, 8) if (ttp * tdp) % e == 0 and arch.num_experts % e == 0])
        iep = rng.choice([e for e in (1, 2, 4, 8) if itp % e == 0 and arch.num_experts % e == 0])
    ok = (heads % ttp == 0 and heads % itp == 0 and kv % ttp == 0 and (itp <= kv or itp % kv == 0) and arch.num_layers % tpp == 0
          and arch.num_layers % ipp == 0 and ttp * tpp * tdp <= 16 and itp * ipp * engines <= 16)
    train = TrainLayout(tp=ttp, pp=tpp, dp=tdp, ep=tep)
    flavour = rng.choice(["vllm", "vllm", "sglang"])
    attn_tp = rng.choice([a for a in (1, 2, 4, 8) if itp % a == 0]) if flavour == "sglang" and rng.random() < 0.4 else 0
    ok = ok and (attn_tp == 0 or (heads % attn_tp == 0 and (attn_tp <= kv or attn_tp % kv == 0)))
    infer = InferLayout(tp=itp, ep=iep, num_engines=engines, engine_name=flavour, pp=ipp, attn_tp=attn_tp, 
                        # a tied head is the embedding tensor, so it is cut the way the embedding is
                        dp_lm_head=bool(attn_tp) and (arch.tie_embeddings or rng.random() < 0.5))
    return ok, arch, train, infer, rng.choice(["round_robin", "spread"])


@pytest.mark.parametrize("seed", range(6))
def test_random_layouts_are_exact(seed):
    rng = random.Random(1000 + seed)
    done = 0
    while done < 12:
        ok, arch, train, infer, pairing = _draw(rng)
        if not ok:
            continue
        label = f"{arch.architecture} h{arch.num_heads}/kv{arch.num_kv_heads} {train.label()} -> {infer.label()} {infer.engine_name} {pairing}"
        job = SimulatedJob(arch, train, infer, dtype=torch.float32)
        job.builder = TransferPlanBuilder(job.infer_world_size, train.world, infer.num_engines, replica_pairing=pairing)
        job.compile_all()
        assert job.check_coverage() == [], label
        job.run_cpu()
        assert job.mismatches() == [], label
        done += 1


def test_random_block_fp8_layouts_through_the_descriptor_tables():
    """Block-aligned small architectures served as fp8: plan, lower, encode, run
    the tables on the host interpreter, compare with the CPU-quantised oracle.
    Quantisation blocks that mix rows of several training ranks go through a
    gathered sender-side buffer; slices that end inside a block are refused with
    NotImplementedError, never mis-executed."""
    from awex_b200.transfer.table_interpreter import HostMemory, run_table

    rng = random.Random(77)
    done = refused = gathered = 0
    while done < 18:
        base = rng.choice(["tiny-llama", "tiny-qwen2", "tiny-qwen3-moe"])
        heads = rng.choice([2, 4, 8])
        kv = rng.choice([k for k in (1, 2, 4, 8) if heads % k == 0 and k <= heads])
        arch = dataclasses.replace(get_arch(base), num_heads=heads, num_kv_heads=kv, head_dim=128, hidden=rng.choice([256, 512]), num_layers=1, vocab=512)
        arch = dataclasses.replace(arch, num_experts=4, expert_ffn=rng.choice([128, 256, 384])) if arch.is_moe else dataclasses.replace(arch, ffn=rng.choice([256, 512, 768]))
        ttp, tdp, itp = rng.choice([1, 2, 2, 4]), rng.choice([1, 2]), rng.choice([1, 2, 4])
        tep = iep = 1
        if arch.is_moe:
            tep = rng.choice([e for e in (1, 2, 4) if (ttp * tdp) % e == 0])
            iep = rng.choice([e for e in (1, 2, 4) if itp % e == 0])
        if heads % ttp or heads % itp or kv % ttp or (itp > kv and itp % kv):
            continue
        train = TrainLayout(tp=ttp, dp=tdp, ep=tep)
        infer = InferLayout(tp=itp, ep=iep, fp8=True, num_engines=rng.choice([1, 2]), engine_name=rng.choice(["vllm", "sglang"]))
        label = f"{base} h{heads}/kv{kv} {train.label()} -> {infer.label()} {infer.engine_name}"
        try:
            job = SimulatedJob(arch, train, infer, dtype=torch.bfloat16)
            job.compile_all()
        except NotImplementedError:
            refused += 1
            continue
        assert job.check_coverage() == [], label
        gathered += any(d.gathers for ds in job.derived.values() for d in ds)
        encoded = job.encode_all(validate=True)
        mem = HostMemory(job.source_tensors() + [p for ms in job.infer_models for m in ms for p in m.parameters()])
        for table, n_tiles, enc in encoded.values():
            run_table(table, n_tiles, mem, enc.row_offsets)
        assert job.mismatches() == [], label
        done += 1
    assert refused < 40
    assert gathered >= 2  # some layouts needed rows of training TP peers for their quantisation blocks
