"""foldjax_b200 - B200 (sm_100a) backend for FoldJAX's Pairformer triangle ops.

Public surface (mirrors the reference's operator interface for this path):

* :func:`foldjax_b200.triangle.triangle_multiplication_forward`
* :func:`foldjax_b200.triangle_attention.triangle_attention_forward`

All arithmetic runs in ``libb200tri.so`` (built by ``python -m foldjax_b200.build``).
"""

__version__ = "0.1.0"
