"""Writes a model description for bin/dnn_benchmark from one of the models of this package.

    python benchmarks/make_dnn_model_csv.py --model resnet50 --batch 64 > models/resnet50.csv
    bin/dnn_benchmark --model models/resnet50.csv --device gpu

One line per module that owns parameters (`layer_index,numel,forward_pass_ns,backward_pass_ns`,
the format of the reference's benchmarks/dnn_benchmark/models/example.csv): `numel` is the
number of gradient elements the layer contributes to the allreduce; the two times are what the
layer's matrix work would take at `--tflops` (2 x parameters x samples floating-point operations
forward, twice that backward; convolutions count every output position). They are estimates
meant to give the benchmark a realistic ratio of computing to communicating, not measurements.
The model is built on the meta device, so no weights are allocated.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def build(name):
    from switchml_b200.models.resnet50 import resnet50
    from switchml_b200.models.vgg19 import vgg19
    from switchml_b200.models.bert_large import bert_large
    with torch.device("meta"):
        if name == "resnet50":
            return resnet50(), (3, 224, 224)
        if name == "vgg19":
            return vgg19(), (3, 224, 224)
        return bert_large(), None


def layers(model, name, batch, seq_len):
    """(numel, forward flops) per module that owns parameters itself, in registration order."""
    rows = []
    hooks = []
    positions = {}

    def hook(mod, inputs, output):
        out = output[0] if isinstance(output, (tuple, list)) else output
        if isinstance(mod, torch.nn.Conv2d):
            positions[mod] = out.shape[-1] * out.shape[-2]
        elif out.dim() >= 3:
            positions[mod] = int(out.numel() // (out.shape[0] * out.shape[-1]))
        else:
            positions[mod] = 1

    leaves = [m for m in model.modules() if any(True for _ in m.parameters(recurse=False))]
    for m in leaves:
        hooks.append(m.register_forward_hook(hook))
    with torch.no_grad(), torch.device("meta"):
        if name == "bert":
            ids = torch.zeros(1, seq_len, dtype=torch.long)
            try:
                model(ids)
            except Exception:  # a model whose forward wants more arguments: fall back to one position per token
                pass
        else:
            model(torch.zeros(1, 3, 224, 224))
    for h in hooks:
        h.remove()
    for m in leaves:
        numel = sum(p.numel() for p in m.parameters(recurse=False))
        per_sample = positions.get(m, seq_len if name == "bert" else 1)
        rows.append((numel, 2.0 * numel * per_sample * batch))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", choices=["resnet50", "vgg19", "bert"], default="resnet50")
    ap.add_argument("--batch", type=int, default=32, help="samples per worker and step")
    ap.add_argument("--seq-len", type=int, default=512, help="tokens per sample (bert)")
    ap.add_argument("--tflops", type=float, default=600.0, help="sustained rate assumed for the layers' matrix work")
    ap.add_argument("--min-ns", type=int, default=2000, help="floor per layer and pass (launch overheads)")
    a = ap.parse_args(argv)
    model, _ = build(a.model)
    print("layer_index, numel, forward_pass_ns, backward_pass_ns")
    for i, (numel, flops) in enumerate(layers(model, a.model, a.batch, a.seq_len)):
        fwd = max(a.min_ns, int(flops / (a.tflops * 1e12) * 1e9))
        print("%d,%d,%d,%d" % (i, numel, fwd, max(a.min_ns, 2 * fwd)))


if __name__ == "__main__":
    main()
