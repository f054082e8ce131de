"""MLIR text export of layer chains (linalg/arith dialect sketch), as the reference's torch/mlir/export.h does."""
import torch.nn as nn


def export(model: nn.Module, input_shape, path: str = None) -> str:
    lines = ["module {", "  func.func @forward(%arg0: tensor<" + "x".join(map(str, input_shape)) + "xf32>) -> tensor<*xf32> {"]
    cur, k, shape = "%arg0", 0, list(input_shape)
    for m in model.modules():
        if isinstance(m, nn.Linear):
            out_shape = shape[:-1] + [m.out_features]
            lines.append(f"    %w{k} = arith.constant dense_resource<w{k}> : tensor<{m.out_features}x{m.in_features}xf32>")
            lines.append(f"    %h{k} = linalg.matmul_transpose_b ins({cur}, %w{k} : tensor<{'x'.join(map(str, shape))}xf32>, "
                         f"tensor<{m.out_features}x{m.in_features}xf32>) -> tensor<{'x'.join(map(str, out_shape))}xf32>")
            cur, shape, k = f"%h{k}", out_shape, k + 1
        elif isinstance(m, (nn.ReLU, nn.Sigmoid, nn.Tanh, nn.GELU, nn.SiLU)):
            lines.append(f"    %a{k} = \"prometorch.{type(m).__name__.lower()}\"({cur}) : (tensor<{'x'.join(map(str, shape))}xf32>) -> "
                         f"tensor<{'x'.join(map(str, shape))}xf32>")
            cur, k = f"%a{k}", k + 1
    lines += [f"    return {cur} : tensor<{'x'.join(map(str, shape))}xf32>", "  }", "}"]
    text = "\n".join(lines)
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text


export_mlir = export                       # the reference's name (torch/mlir/export.h)
