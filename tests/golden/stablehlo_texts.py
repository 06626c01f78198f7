"""StableHLO-subset texts used by the importer fixtures and tests (written for this
repository: a dense decoder layer, a MoE decoder layer and a graph without the fused-QKV
pattern)."""

DECODER_TEXT = """module {
  func.func @layer(%x: tensor<4x16xf32>, %n1w: tensor<16xf32>, %q_w: tensor<16x16xf32>,
      %k_w: tensor<16x8xf32>, %v_w: tensor<16x8xf32>, %o_w: tensor<16x16xf32>,
      %n2w: tensor<16xf32>, %g_w: tensor<16x32xf32>, %u_w: tensor<16x32xf32>,
      %d_w: tensor<32x16xf32>) -> tensor<4x16xf32> {
    %h0 = stablehlo.custom_call @RmsNorm(%x, %n1w) : tensor<4x16xf32>
    %qp = stablehlo.dot_general %h0, %q_w : tensor<4x16xf32>
    %kp = stablehlo.dot_general %h0, %k_w : tensor<4x8xf32>
    %vp = stablehlo.dot_general %h0, %v_w : tensor<4x8xf32>
    %qr = stablehlo.custom_call @RoPE(%qp) : tensor<4x16xf32>
    %kr = stablehlo.custom_call @RoPE(%kp) : tensor<4x8xf32>
    %ao = stablehlo.dot_general %qr, %o_w : tensor<4x16xf32>
    %r1 = stablehlo.add %ao, %x : tensor<4x16xf32>
    %h1 = stablehlo.custom_call @RmsNorm(%r1, %n2w) : tensor<4x16xf32>
    %gp = stablehlo.dot_general %h1, %g_w : tensor<4x32xf32>
    %up = stablehlo.dot_general %h1, %u_w : tensor<4x32xf32>
    %sw = stablehlo.custom_call @SwiGLU(%gp, %up) : tensor<4x32xf32>
    %dn = stablehlo.dot_general %sw, %d_w : tensor<4x16xf32>
    %y = stablehlo.add %dn, %r1 : tensor<4x16xf32>
    return %y
  }
}
"""

MOE_TEXT = """module {
  func.func @layer_moe(%x: tensor<4x16xf32>, %n1w: tensor<16xf32>, %q_w: tensor<16x16xf32>,
      %k_w: tensor<16x8xf32>, %v_w: tensor<16x8xf32>, %o_w: tensor<16x16xf32>,
      %n2w: tensor<16xf32>, %r_w: tensor<16x4xf32>) -> tensor<4x16xf32> {
    %h0 = stablehlo.custom_call @RmsNorm(%x, %n1w) : tensor<4x16xf32>
    %qp = stablehlo.dot_general %h0, %q_w : tensor<4x16xf32>
    %kp = stablehlo.dot_general %h0, %k_w : tensor<4x8xf32>
    %vp = stablehlo.dot_general %h0, %v_w : tensor<4x8xf32>
    %qr = stablehlo.custom_call @RoPE(%qp) : tensor<4x16xf32>
    %kr = stablehlo.custom_call @RoPE(%kp) : tensor<4x8xf32>
    %ao = stablehlo.dot_general %qr, %o_w : tensor<4x16xf32>
    %r1 = stablehlo.add %ao, %x : tensor<4x16xf32>
    %h1 = stablehlo.custom_call @RmsNorm(%r1, %n2w) : tensor<4x16xf32>
    %logits = stablehlo.dot_general %h1, %r_w : tensor<4x4xf32>
    %ffn = stablehlo.custom_call @MoeFFN(%h1, %logits) : tensor<4x16xf32>
    %y = stablehlo.add %ffn, %r1 : tensor<4x16xf32>
    return %y
  }
}
"""

NO_QKV_TEXT = """func.func @f(%x: tensor<4x16xf32>, %w: tensor<16x16xf32>) -> tensor<4x16xf32> {
    %a = stablehlo.dot_general %x, %w : tensor<4x16xf32>
    %b = stablehlo.custom_call @RoPE(%a) : tensor<4x16xf32>
    return %b
}
"""



def dense_decoder_text(rows, hidden, kv_width, intermediate):
    """The dense layer text above with other extents."""
    return (DECODER_TEXT.replace("4x16xf32", f"{rows}x{hidden}xf32").replace("16x16xf32", f"{hidden}x{hidden}xf32")
            .replace("16x8xf32", f"{hidden}x{kv_width}xf32").replace("4x8xf32", f"{rows}x{kv_width}xf32")
            .replace("16x32xf32", f"{hidden}x{intermediate}xf32").replace("4x32xf32", f"{rows}x{intermediate}xf32")
            .replace("32x16xf32", f"{intermediate}x{hidden}xf32").replace("tensor<16xf32>", f"tensor<{hidden}xf32>"))
