"""Whole-model launcher with the reference's command line (inference-engine/run_model.py:7-13):

    python run_model.py --transformer_config_file configs/vit_base_model.yaml
                        [--model_weight_file weights.npz] [--need_compile] [--need_breakdown] [--tune]

layer_num encoder layers back to back (transformer_model.cpp:13-49).  Weights come from a
converted .npz checkpoint when the file exists, else random (test_transformer.cpp:470-489).
"""
import run_layer

if __name__ == '__main__':
    run_layer.run(run_layer.parse_args(), whole_model=True)
