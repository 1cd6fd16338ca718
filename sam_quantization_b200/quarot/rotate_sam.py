"""``rotate_sam`` — the QuaRot recipe for the SAM image encoder (quarot/rotate_sam.py:67-101)."""
from __future__ import annotations

from . import hadamard_utils, rotation_utils, utils


def rotate_sam(sam_model, args, rtn_ro_config, decoder=False, fuse_online_rotation=True):
    """Rotate the encoder's weights, wrap every Linear in an ``ActQuantWrapper`` configured from
    ``rtn_ro_config`` and flag the online transforms by layer name:

    * ``...mlp.lin2``  -> ``online_full_had`` of size lin2.in_features   (:78-87)
    * ``image_encoder...proj`` -> ``online_partial_had`` across heads, ``had_dim = hidden // heads`` (:88-94)

    ``args`` carries ``hidden_size_image_en``, ``num_attention_head_image_en``, ``rotate_mode``,
    ``device``, ``seed`` and ``fp32_had`` (see ``utils.parser_gen``).  With
    ``fuse_online_rotation`` and ``rotate_mode == "hadamard"`` the online ``x @ Q`` in front of qkv
    and lin1 is folded into those layers' quantization kernel as a sign flip plus fast transform
    (the same matrix); otherwise it stays a dense matmul as in the reference.  The mask-decoder
    branch (``decoder=True``) needs the SAM decoder and is not provided."""
    if decoder:
        raise NotImplementedError("rotating the mask decoder needs the SAM decoder, which this package does not host")
    sam_model.eval()
    Q = rotation_utils.get_orthogonal_matrix(args.hidden_size_image_en, args.rotate_mode, device=args.device, seed=args.seed)
    rotation_utils.rotate_model(sam_model, Q, None, args)
    utils.cleanup_memory(verbos=True)
    utils.add_actquant(sam_model, rtn_ro_config=rtn_ro_config)
    qlayers = utils.find_qlayers(sam_model)
    signs = None
    if fuse_online_rotation and args.rotate_mode == "hadamard":
        signs = hadamard_utils.random_hadamard_signs(args.hidden_size_image_en, args.seed).to(args.device)
        pre_hadK, pre_K = hadamard_utils.get_hadK(args.hidden_size_image_en)
        if pre_hadK is not None:
            pre_hadK = pre_hadK.to(args.device)
    for name, layer in qlayers.items():
        if not isinstance(layer, utils.ActQuantWrapper):
            continue
        if "lin2" in name and "final_attn" not in name and "image_encoder" in name:
            width = sam_model.image_encoder.blocks[0].mlp.lin2.weight.shape[1]
            had_K, K = hadamard_utils.get_hadK(width)
            layer.online_full_had = True
            layer.had_K = None if had_K is None else had_K.to(args.device)
            layer.K = K
            layer.fp32_had = args.fp32_had
        if "image_encoder" in name and "proj" in name:
            had_K, K = hadamard_utils.get_hadK(args.num_attention_head_image_en)
            layer.online_partial_had = True
            layer.had_K = None if had_K is None else had_K.to(args.device)
            layer.K = K
            layer.had_dim = args.hidden_size_image_en // args.num_attention_head_image_en
            layer.fp32_had = args.fp32_had
        if signs is not None and (name.endswith("attn.qkv") or name.endswith("mlp.lin1")):
            layer.set_pre_rotation(signs, pre_hadK, pre_K)
    return qlayers
