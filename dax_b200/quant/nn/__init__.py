from . import dynamic, quantized
