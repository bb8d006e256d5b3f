// Name -> factory registry of operators, as in the reference (utils/operator_registry.h:27-69):
// a mutex-guarded singleton, RegisterOperator that refuses duplicates, CreateOperator that returns
// nullptr for an unknown name, and the REGISTER_OPERATOR static-initialiser macro.
#ifndef CATCCOS_B200_HOST_OPERATOR_REGISTRY_H
#define CATCCOS_B200_HOST_OPERATOR_REGISTRY_H

#include <mutex>

#include "catccos_operator.h"

class OperatorRegistry {
public:
    static OperatorRegistry& Instance()
    {
        static OperatorRegistry registry;
        return registry;
    }

    bool RegisterOperator(const std::string& op_type, OperatorCreator creator)
    {
        std::lock_guard<std::mutex> guard(mutex_);
        return creators_.emplace(op_type, std::move(creator)).second;
    }

    std::unique_ptr<CatccosOperator> CreateOperator(const std::string& op_type)
    {
        std::lock_guard<std::mutex> guard(mutex_);
        auto found = creators_.find(op_type);
        return found == creators_.end() ? nullptr : found->second();
    }

private:
    OperatorRegistry() = default;
    std::unordered_map<std::string, OperatorCreator> creators_;
    std::mutex mutex_;
};

#define REGISTER_OPERATOR(op_type, op_class)                                                              \
    class op_class;                                                                                       \
    namespace {                                                                                           \
    struct op_class##_registrar {                                                                         \
        op_class##_registrar()                                                                            \
        {                                                                                                 \
            OperatorRegistry::Instance().RegisterOperator(                                                \
                op_type, []() -> std::unique_ptr<CatccosOperator> { return std::make_unique<op_class>(); }); \
        }                                                                                                 \
    };                                                                                                    \
    static op_class##_registrar op_class##_instance;                                                      \
    }

#endif  // CATCCOS_B200_HOST_OPERATOR_REGISTRY_H
