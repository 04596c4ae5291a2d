"""Accuracy of the per-site choices on synthetic activations (CPU oracle only): NVFP4 activations
against bf16 activations over NVFP4 weights, on Gaussian and on heavy-tailed inputs. The numbers
back the site policy: which linears may take FP4 activations and where an outlier-aware fallback
(bf16 activations over FP4 weights, the analogue of the reference's dense-activation sites,
thinfer-models/src/common/block.rs:458-479) is the safer choice."""
import numpy as np

import oracle as O
from conftest import rel_fro

M, K, N = 96, 1024, 256


def _errors(a_f32, w):
    """Relative Frobenius error against the unquantised f64 product, for three policies."""
    a = O.f32_to_bf16(a_f32)
    af = O.bf16_to_f32(a)
    exact = af.astype(np.float64) @ w.astype(np.float64).T
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    fp4_both = O.bf16_to_f32(O.linear(a, ga, wc, ws, gw))                     # FP4 activations x FP4 weights
    fp4_w = O.bf16_to_f32(O.linear(a, ga, wc, ws, gw, quantize_a=False))      # bf16 activations x FP4 weights
    bf16 = O.bf16_to_f32(O.f32_to_bf16((af.astype(np.float64) @ O.bf16_to_f32(O.f32_to_bf16(w)).astype(np.float64).T).astype(np.float32)))
    return rel_fro(fp4_both, exact), rel_fro(fp4_w, exact), rel_fro(bf16, exact)


def test_fp4_activation_error_on_gaussian_and_heavy_tailed_inputs():
    w = (O.gaussian(N * K, 71) * np.float32(0.02)).reshape(N, K)
    gauss = O.gaussian(M * K, 72).reshape(M, K)
    # heavy tails: a few channels carry 30x outliers, as DiT activations do after modulation
    heavy = gauss.copy()
    heavy[:, ::128] *= np.float32(30.0)
    e_g, e_h = _errors(gauss, w), _errors(heavy, w)
    # ordering of the policies
    assert e_g[2] < e_g[1] < e_g[0] and e_h[2] < e_h[1] < e_h[0]
    # two-level scaling (E4M3 per 16 + f32 per tensor) keeps FP4 activations usable on both inputs ...
    assert e_g[0] < 0.16 and e_h[0] < 0.16
    # ... the weights' quantisation is most of the error, FP4 activations add less than a factor 1.6
    assert e_g[0] < 1.6 * e_g[1] and e_h[0] < 1.6 * e_h[1]
    # outliers confined to their own 16-blocks do not spoil the rest: the heavy-tailed error stays within
    # 1.5x of the Gaussian one (a per-tensor int8-style scale would lose the small channels entirely)
    assert e_h[0] < 1.5 * e_g[0]
    print("policy study (rel. Frobenius error vs f64): gaussian fp4xfp4 %.4f bf16xfp4 %.4f bf16 %.5f | heavy-tailed %.4f %.4f %.5f"
          % (e_g + e_h))
