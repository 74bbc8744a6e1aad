"""Library-independent dtype names with torch / numpy conversions (parity: `fast_llm/engine/config_utils/data_type.py`)."""

import enum


class DataType(str, enum.Enum):
    float64 = "float64"
    float32 = "float32"
    float16 = "float16"
    bfloat16 = "bfloat16"
    int64 = "int64"
    int32 = "int32"
    int16 = "int16"
    int8 = "int8"
    uint8 = "uint8"
    uint16 = "uint16"
    uint32 = "uint32"
    uint64 = "uint64"
    bool = "bool"

    @classmethod
    def _missing_(cls, value):
        if isinstance(value, str):
            alt = _ALTERNATE_NAMES.get(value.lower().replace("torch.", "").replace("numpy.", "").replace("np.", ""))
            if alt is not None:
                return cls(alt)
        return None

    @property
    def torch(self):
        import torch

        return getattr(torch, self.value)

    @classmethod
    def from_torch(cls, dtype) -> "DataType":
        return cls(str(dtype).replace("torch.", ""))

    @property
    def numpy(self):
        import numpy as np

        if self == DataType.bfloat16:
            raise ValueError("numpy has no bfloat16")
        return np.dtype(self.value if self != DataType.bool else "bool_").type

    @classmethod
    def from_numpy(cls, dtype) -> "DataType":
        import numpy as np

        return cls(np.dtype(dtype).name)

    @property
    def itemsize(self) -> int:
        return {"float64": 8, "float32": 4, "float16": 2, "bfloat16": 2, "int64": 8, "int32": 4, "int16": 2, "int8": 1,
                "uint8": 1, "uint16": 2, "uint32": 4, "uint64": 8, "bool": 1}[self.value]

    @property
    def is_float(self) -> "bool":
        return self.value.startswith(("float", "bfloat"))


_ALTERNATE_NAMES = {
    "fp64": "float64", "double": "float64", "fp32": "float32", "float": "float32", "fp16": "float16", "half": "float16",
    "bf16": "bfloat16", "long": "int64", "int": "int32", "short": "int16", "byte": "uint8",
}


def get_unsigned_integer_type(max_size: int) -> DataType:
    for dt, bits in ((DataType.uint8, 8), (DataType.uint16, 16), (DataType.uint32, 32)):
        if max_size < 2**bits:
            return dt
    return DataType.int64
