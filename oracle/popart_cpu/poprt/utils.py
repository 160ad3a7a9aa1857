def convert_float_to_uint8(array, fmt="F143", scale=-1):
    raise NotImplementedError("Graphcore F143 conversion lives in the closed poprt wheel; the FP8 path is oracle-defined as OCP E4M3")
