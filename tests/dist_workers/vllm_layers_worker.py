"""Runs in its own process (vLLM keeps process-wide state): build vLLM's parallel linear layers on the CPU, convert
them with the package's vLLM adapter, compare with the dense product, and install the engine patches on the installed
vLLM's classes.  Prints ``OK`` on success."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    port = sys.argv[1] if len(sys.argv) > 1 else "29641"
    from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config
    from vllm.distributed import init_distributed_environment, initialize_model_parallel
    with set_current_vllm_config(VllmConfig(device_config=DeviceConfig(device="cpu"))):
        init_distributed_environment(world_size=1, rank=0, distributed_init_method=f"tcp://127.0.0.1:{port}",
                                     local_rank=0, backend="gloo")
        initialize_model_parallel(1, 1)
        from vllm.model_executor.layers.linear import (MergedColumnParallelLinear, QKVParallelLinear,
                                                       RowParallelLinear)
        from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead

        class Block(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.qkv_proj = QKVParallelLinear(128, 32, 4, 2, bias=False)
                self.o_proj = RowParallelLinear(128, 128, bias=False)
                self.gate_up_proj = MergedColumnParallelLinear(128, [256, 256], bias=False)
                self.lm_head = ParallelLMHead(512, 128)

        torch.manual_seed(0)
        blk = Block()
        dense = {}
        for name, mod in blk.named_children():
            mod.weight.data.normal_(0, 0.05)
            dense[name] = mod.weight.data.clone().float()

        from ipex_llm_b200.ops.linear import LowBitLinear
        from ipex_llm_b200.vllm.model_convert import _get_logits, _ipex_llm_convert, _PATCHED, convert_vllm_model
        low = convert_vllm_model(blk, "sym_int8", torch.float32)
        x = torch.randn(5, 128)
        for name in ("qkv_proj", "o_proj", "gate_up_proj"):
            mod = getattr(low, name)
            assert isinstance(mod, LowBitLinear), (name, type(mod))
            out = mod(x)
            assert isinstance(out, tuple) and out[1] is None, name        # vLLM layers return (output, bias)
            want = x @ dense[name].t()
            cos = torch.nn.functional.cosine_similarity(out[0].float().flatten(), want.flatten(), dim=0).item()
            assert cos > 0.999, (name, cos)
        assert isinstance(low.lm_head, LowBitLinear)

        class Proc:
            org_vocab_size = 500
        logits = _get_logits(Proc(), x, low.lm_head, None)
        want = (x @ dense["lm_head"].t())[:, :500]
        assert logits.shape == (5, 500)
        assert torch.nn.functional.cosine_similarity(logits.float().flatten(), want.flatten(), dim=0).item() > 0.999

        # the patches land on the classes of the installed vLLM
        from vllm.model_executor.layers.logits_processor import LogitsProcessor
        from vllm.v1.worker.gpu_model_runner import GPUModelRunner
        before = GPUModelRunner.load_model
        _ipex_llm_convert("sym_int4")
        assert GPUModelRunner in _PATCHED and GPUModelRunner.load_model is not before
        assert LogitsProcessor._get_logits is _get_logits

        # the patched loader converts whatever the original loader left in ``self.model``
        class Runner:
            model = None
            model_config = type("C", (), {"dtype": torch.float32})()
        fresh = Block()
        for mod in fresh.children():
            mod.weight.data.normal_(0, 0.05)
        _PATCHED[GPUModelRunner], saved = (lambda self, *a, **k: setattr(self, "model", fresh)), _PATCHED[GPUModelRunner]
        try:
            r = Runner()
            # the wrapper captured the original at patch time; exercise the same logic through a second patch target
            from ipex_llm_b200.vllm import model_convert as mc

            class Target:
                def load_model(self, load_dummy_weights=False):
                    self.model = fresh
            mc.patch_runner_class(Target, "sym_int8")
            t = Target()
            t.model_config = r.model_config
            t.load_model()
            assert isinstance(t.model.qkv_proj, LowBitLinear)
        finally:
            _PATCHED[GPUModelRunner] = saved
        # the engine classes are subclasses of the installed vLLM's and hand every other argument through
        from vllm.engine.llm_engine import LLMEngine
        from vllm.v1.engine.async_llm import AsyncLLM
        from ipex_llm_b200.vllm import engine as eng
        assert issubclass(eng.IPEXLLMLLMEngine, LLMEngine) and issubclass(eng.IPEXLLMAsyncV1Engine, AsyncLLM)
        import vllm
        assert issubclass(eng.IPEXLLMClass, vllm.LLM)
        seen = {}
        orig = LLMEngine.__dict__["from_engine_args"]
        LLMEngine.from_engine_args = classmethod(lambda cls, engine_args, *a, **k: seen.update(cls=cls, args=engine_args, kw=k))
        try:
            eng.IPEXLLMLLMEngine.from_engine_args("ARGS", load_in_low_bit="fp8", usage_context="ctx")
        finally:
            LLMEngine.from_engine_args = orig
        assert seen["cls"] is eng.IPEXLLMLLMEngine and seen["args"] == "ARGS" and seen["kw"] == {"usage_context": "ctx"}
        assert os.environ.get("VLLM_ENABLE_V1_MULTIPROCESSING") == "0"
        # the server entry point: one extra flag on vLLM's own parser, then vLLM's run_server
        from ipex_llm_b200.vllm.entrypoints.openai import api_server as srv
        import vllm.entrypoints.openai.api_server as vsrv
        try:
            ns = srv.make_parser().parse_args(["--model", "some/dir", "--load-in-low-bit", "fp8", "--port", "8123"])
            assert ns.load_in_low_bit == "fp8" and ns.model == "some/dir" and ns.port == 8123
        except RuntimeError as e:
            # vLLM computes its flag defaults from the device it detects; a host without one cannot build the parser
            assert "device type" in str(e), e
            import argparse

            def stand_in():
                p = argparse.ArgumentParser()
                p.add_argument("--model")
                p.add_argument("--load-in-low-bit", default="sym_int4")
                return p
            srv.make_parser = stand_in
        ran = {}

        async def fake_run_server(args, **kw):
            ran["low_bit"] = args.load_in_low_bit
        real, vsrv.run_server = vsrv.run_server, fake_run_server
        try:
            srv.main(["--model", "some/dir", "--load-in-low-bit", "nf4"])
        finally:
            vsrv.run_server = real
        assert ran == {"low_bit": "nf4"}
        from ipex_llm_b200.vllm.xpu.engine import IPEXLLMClass as viaxpu
        assert viaxpu is eng.IPEXLLMClass
    print("OK")


if __name__ == "__main__":
    main()
