"""torchao.prototype: the quant_llm (FPx) and hqq (HQQ-layout int4) parts."""
