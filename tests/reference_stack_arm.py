"""One arm of the whole-stack check: the reference's OWN layer and trainer, unmodified, on top of either its
Triton ops (``--ops triton``) or the CUDA ops of this repository (``--ops cuda``, swapped in by
``palimpsa_b200.install_as_palimpsa_ops()`` before anything of the reference is imported).

    python tests/reference_stack_arm.py --ops cuda|triton --out RESULT.pt [--nano-iters 100]

Runs, on cuda:0, from the unmodified working copy under ``oracle/_ref/``:

1. ``palimpsa.layers.palimpsa.Palimpsa`` (palimpsa/layers/palimpsa.py:33-348) in training mode under bf16
   autocast: forward (the layer's chunk call, :309) and backward; output, input gradient and a few parameter
   gradients are saved.
   The same for ``palimpsa.layers.meta_mamba2.MetaMamba2`` (palimpsa/layers/meta_mamba2.py:35-376), which calls
   the ops with raw (unnormalised) q/k, ``scale=1.0`` and d_k = 32, d_v = 128 (:333).
2. the Palimpsa layer in eval mode with an FLA ``Cache``: a 100-token prefill (chunk mode, final states into the
   cache) followed by three single-token steps (the layer's fused-recurrent call with cached states, :317).
3. ``train_nano.py`` itself (train_nano.py:1-185), executed with ``runpy`` from the copy's folder with
   ``--max_iters N``; its printed losses and per-50-iteration times are parsed from its output.

4. a packed variable-length TRAINING STEP of the reference's ``PalimpsaForCausalLM`` in the 170M model's shape
   (config/palimpsa_170M.json: 16 heads of d_k = d_v = 48; 4 of its 19 layers), the way its Flame recipe feeds it
   (README.md:135-158: one packed row, ``cu_seqlens`` through the model's kwargs to every layer,
   palimpsa/models/palimpsa/modeling_palimpsa.py:255-262): loss, a few gradients and the step time.

Writes everything into ``--out`` (torch.save).  The parent test compares the two arms' files.
"""
import argparse
import contextlib
import io
import os
import re
import runpy
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", choices=["cuda", "triton"], required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--nano-iters", type=int, default=100)
    ap.add_argument("--nano-batch", type=int, default=32)
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    import torch
    if a.ops == "cuda":
        import palimpsa_b200
        palimpsa_b200.install_as_palimpsa_ops()
    from fla.models.utils import Cache
    from palimpsa.layers import palimpsa as layer_mod
    res = {"ops": a.ops, "chunk_op_module": layer_mod.chunk_palimpsa.__module__,
           "fused_op_module": layer_mod.fused_recurrent_palimpsa.__module__}
    dev = torch.device("cuda", 0)

    # ---- 1. training-mode forward / backward through the reference layer ---------------------------------
    torch.manual_seed(0)
    layer = layer_mod.Palimpsa(hidden_size=256, head_dim=64, num_heads=4, expand_v=2, layer_idx=0).to(dev)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(2, 192, 256, generator=gen).to(dev).requires_grad_(True)
    w = torch.randn(2, 192, 256, generator=gen).to(dev)
    layer.train()
    with torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
        y, _, _ = layer(x)
    (y.float() * w).sum().backward()
    res["train_out"] = y.detach().float().cpu()
    res["train_dx"] = x.grad.float().cpu()
    for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "b_proj.weight", "dt_proj.weight", "A_log",
              "dt_bias", "b_scale", "D", "g_proj.weight"):
        p = dict(layer.named_parameters())[n]
        res["train_grad_" + n] = p.grad.float().cpu()

    # ---- 1b. the MetaMamba2 layer: raw q/k, scale = 1, d_k = 32 / d_v = 128 --------------------------------------
    from palimpsa.layers import meta_mamba2 as mm2_mod
    res["mm2_chunk_op_module"] = mm2_mod.chunk_palimpsa.__module__
    torch.manual_seed(2)
    mm2 = mm2_mod.MetaMamba2(num_heads=4, head_dim=128, hidden_size=256, state_size=32, expand=2, layer_idx=0,
                             init_diagnosis=False).to(dev)
    x2 = torch.randn(2, 160, 256, generator=gen).to(dev).requires_grad_(True)
    w2 = torch.randn(2, 160, 256, generator=gen).to(dev)
    mm2.train()
    with torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
        y2, _, _ = mm2(x2)
    (y2.float() * w2).sum().backward()
    res["mm2_out"] = y2.detach().float().cpu()
    res["mm2_dx"] = x2.grad.float().cpu()
    for n, prm in mm2.named_parameters():
        if prm.grad is not None:
            res["mm2_grad_" + n] = prm.grad.float().cpu()
    del mm2

    # ---- 2. eval: prefill with cache, then single-token decode steps -----------------------------------------
    layer.eval()
    xs = torch.randn(3, 103, 256, generator=gen).to(dev)
    cache = Cache()
    outs = []
    with torch.no_grad(), torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
        y, _, cache = layer(xs[:, :100], past_key_values=cache, use_cache=True)
        outs.append(y)
        for t in range(100, 103):
            y, _, cache = layer(xs[:, t:t + 1], past_key_values=cache, use_cache=True)
            outs.append(y)
    res["decode_out"] = torch.cat(outs, 1).float().cpu()
    mu, I = cache[0]["recurrent_state"]
    res["decode_final_mu"], res["decode_final_I"] = mu.float().cpu(), I.float().cpu()
    del layer, cache
    torch.cuda.synchronize()

    # ---- 3. the reference's trainer, as it is ---------------------------------------------------------------
    if a.nano_iters > 0:
        argv, cwd = sys.argv, os.getcwd()
        buf = io.StringIO()
        t0 = time.time()
        try:
            os.chdir(REF)
            sys.argv = ["train_nano.py", "--model", "palimpsa", "--max_iters", str(a.nano_iters), "--batch_size",
                        str(a.nano_batch), "--n_layer", "4", "--device", "cuda"]
            with contextlib.redirect_stdout(buf):
                runpy.run_path(os.path.join(REF, "train_nano.py"), run_name="__main__")
        finally:
            os.chdir(cwd)
            sys.argv = argv
        text = buf.getvalue()
        res["nano_stdout"] = text
        res["nano_wall_s"] = time.time() - t0
        res["nano_iter_loss"] = {int(m.group(1)): float(m.group(2))
                                 for m in re.finditer(r"iter (\d+): loss ([0-9.]+)", text)}
        res["nano_iter_ms"] = {int(m.group(1)): float(m.group(2))
                               for m in re.finditer(r"iter (\d+): loss [0-9.]+, time ([0-9.]+)ms", text)}
        res["nano_eval"] = {int(m.group(1)): (float(m.group(2)), float(m.group(3)))
                            for m in re.finditer(r"step (\d+): train loss ([0-9.]+), val loss ([0-9.]+)", text)}
    # ---- 4. packed variable-length training step of the 170M-shaped model ------------------------------------
    try:
        import json
        from palimpsa.models.palimpsa.configuration_palimpsa import PalimpsaConfig
        from palimpsa.models.palimpsa.modeling_palimpsa import PalimpsaForCausalLM
        with open(os.path.join(REF, "config", "palimpsa_170M.json")) as f:
            cfg = {k: v for k, v in json.load(f).items() if k not in ("architectures", "auto_map", "model_type")}
        # 4 layers; untied embeddings (the installed transformers release rejects the reference's list-typed
        # _tied_weights_keys when the config ties them -- a packaging matter, not part of the path under test)
        cfg.update(num_hidden_layers=4, use_cache=False, tie_word_embeddings=False)
        torch.manual_seed(3)
        model = PalimpsaForCausalLM(PalimpsaConfig(**cfg)).to(dev)
        model.train()
        T = 16384
        g2 = torch.Generator().manual_seed(4)
        lens, tot = [], 0
        while tot < T:                                       # documents of 128 .. 4096 tokens, as the recipe packs them
            n = min(int(torch.randint(128, 4097, (1,), generator=g2).item()), T - tot)
            lens.append(n)
            tot += n
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        ids = torch.randint(0, cfg["vocab_size"], (1, T), generator=g2).to(dev)

        def step():
            model.zero_grad(set_to_none=True)
            with torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
                out = model(ids, labels=ids, cu_seqlens=cu)
            out.loss.backward()
            return out.loss

        loss = step()
        torch.cuda.synchronize()
        res["varlen_loss"] = float(loss)
        params = dict(model.named_parameters())
        for n in ("model.embeddings.weight", "model.layers.0.attn.q_proj.weight", "model.layers.0.attn.A_log",
                  "model.layers.0.attn.b_proj.weight", "model.layers.3.attn.dt_bias", "model.layers.3.attn.v_proj.weight"):
            if n in params and params[n].grad is not None:
                res["varlen_grad_" + n] = params[n].grad.float().cpu()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            step()
        e1.record()
        torch.cuda.synchronize()
        res["varlen_step_ms"] = e0.elapsed_time(e1) / 3
        res["varlen_documents"] = len(lens)
    except Exception as e:                                    # noqa: BLE001  (reported by the parent test)
        import traceback
        res["varlen_error"] = traceback.format_exc()[-1500:]
    torch.save(res, a.out)
    print(f"{a.ops} arm done: chunk op from {res['chunk_op_module']}")


if __name__ == "__main__":
    main()
