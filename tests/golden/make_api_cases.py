"""Distils the reference's phase-1 behaviour table for aclnnQuantMatmulV5 into `api_v5_cases.json`.

Source: matmul/quant_batch_matmul_v4/tests/ut/op_host/test_aclnn_quant_matmul_v5_api.csv of the reference (the rows its
own op_api unit test feeds to aclnnQuantMatmulV5GetWorkspaceSize with null device addresses, together with the expected
status). Only the rows for the current NPU generation (socVersion Ascend950) are kept; tensor construction follows the
reference test driver (test_aclnn_quant_matmul_v5_api.cpp:186-300: an empty shape means the argument is nullptr, x1/x2
use the listed strides, every other tensor is dense).

    python tests/golden/make_api_cases.py
"""
import csv
import json
import os

REF = os.environ.get("OPSNN_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference"))
SRC = os.path.join(REF, "matmul/quant_batch_matmul_v4/tests/ut/op_host/test_aclnn_quant_matmul_v5_api.csv")
HERE = os.path.dirname(os.path.abspath(__file__))


def ints(s):
    return [int(v) for v in s.split()] if s.strip() else []


def main():
    cases = []
    with open(SRC, newline="") as fh:
        for row in csv.DictReader(fh):
            if row["socVersion"] != "Ascend950":
                continue
            c = {"name": row["caseName"], "expect": row["expectRet"],
                 "transposeX1": row["transposeX1"].strip().lower() == "true",
                 "transposeX2": row["transposeX2"].strip().lower() == "true",
                 "groupSize": int(row["groupSize"] or 0), "x1Format": row["x1Format"] or "ACL_FORMAT_ND",
                 "x2Format": row["x2Format"] or "ACL_FORMAT_ND", "tensors": {}}
            for key, shape_col, type_col, stride_col in (
                    ("x1", "x1Shape", "x1Type", "x1Stride"), ("x2", "x2Shape", "x2Type", "x2Stride"),
                    ("x2Scale", "scaleShape", "scaleType", None), ("x2Offset", "offsetShape", "offsetType", None),
                    ("x1Scale", "pertokenScaleShape", "pertokenType", None), ("bias", "biasShape", "biasType", None),
                    ("yScale", "yScaleShape", "yScaleType", None), ("x1Offset", "x1OffsetShape", "x1OffsetType", None),
                    ("yOffset", "yOffsetShape", "yOffsetType", None), ("out", "outShape", "outType", None)):
                shape = ints(row[shape_col])
                if not shape:
                    continue
                t = {"shape": shape, "dtype": row[type_col]}
                if stride_col and row[stride_col].strip():
                    t["strides"] = ints(row[stride_col])
                storage = row.get(shape_col.replace("Shape", "StorageShape"), "") if key in ("x1", "x2") else ""
                if storage and storage.strip():
                    t["storage_shape"] = ints(storage)
                c["tensors"][key] = t
            cases.append(c)
    with open(os.path.join(HERE, "api_v5_cases.json"), "w") as fh:
        json.dump(cases, fh, indent=0)
    print(len(cases), "cases")


if __name__ == "__main__":
    main()
