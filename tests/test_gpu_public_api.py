"""Writer and reader in one process on one GPU, through the public API: the
co-resident deployment (training rank and inference worker share the device).
Checks bitwise results, validation with a poisoned parameter, and that a
second update after an in-place "optimizer step" lands."""

import threading

import pytest
import torch

pytestmark = pytest.mark.gpu


def _prepare_both(writer, reader):
    errors = []

    def run(fn):
        try:
            torch.cuda.set_device(0)
            fn()
        except BaseException as exc:
            errors.append(exc)

    threads = [threading.Thread(target=run, args=(reader.prepare,)), threading.Thread(target=run, args=(writer.prepare,))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    if errors:
        raise errors[0]


@pytest.mark.parametrize("arch_name", ["tiny-qwen2", "tiny-qwen3-moe"])
def test_colocated_update_through_public_api(arch_name):
    from awex_b200 import NCCLWeightsWriter, WeightsReader
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine, SyntheticTrainEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos, train_rank_infos

    torch.cuda.set_device(0)
    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    arch = get_arch(arch_name)
    train = SyntheticTrainEngine(arch, train_rank_infos()[0], addr, dtype=torch.bfloat16, device="cuda")
    # the engine has loaded the same weights training holds, so step 1 can be
    # validated against the engine's own contents (recorded, cleared, compared)
    infer = SyntheticInferenceEngine(arch, InferLayout(tp=1), infer_rank_infos()[0], addr, dtype=torch.bfloat16, device="cuda",
                                     zero=False, weights_validation_steps=1)
    writer, reader = NCCLWeightsWriter(train), WeightsReader(infer)
    writer.initialize()
    reader.initialize()
    _prepare_both(writer, reader)
    for step in (1, 2):
        if step == 2:
            train.regenerate(step=2)
        reader.begin_update(step)
        writer.write_weights(step_id=step)
        reader.finish_update(step)
        if step == 1:
            assert reader.last_validation_failed == []
        assert infer.mismatches(step=0 if step == 1 else 2) == []
    assert infer.schedulers[0].flushes == 2
    writer.close()
    server.stop()
