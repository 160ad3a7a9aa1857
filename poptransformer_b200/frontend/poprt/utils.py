def convert_float_to_uint8(*args, **kwargs):
    """poprt.utils.convert_float_to_uint8(w, 'F143', -1) (precision_strategy.py:50) produces Graphcore F143 bytes, whose
    exponent bias and range differ from OCP E4M3; the arithmetic is closed, so the 'fp8' / 'fp8_weight' precisions of the
    reference are not driven through this front end."""
    raise NotImplementedError("Graphcore F143 quantisation is not available on this backend: quantise with "
                              "poptransformer_b200.quant.quantize_fp8 (OCP E4M3, per-tensor scale) and use the ChatGLM2 FP8 decoder")
